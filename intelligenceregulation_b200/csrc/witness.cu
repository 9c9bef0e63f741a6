// Witness weight products (hashline/src/gpu/metal.rs:4646-4680 witness_product; private_block/witness.rs:979-991): the one
// dense contraction of the system, exact integers: int16 activations times int8 weights into int64.
//
//   k_wp_pack      x (int64, row stride xs) -> two byte planes per 128-token tile: hi = x >> 8 (signed), lo = x & 255
//                  (unsigned), K padded with zeros to a multiple of 128; an activation outside int16 raises the flag
//   k_wp_repack    weights the product kernel cannot read in place (in_out layout, or K not a multiple of 128) -> rows of Kp bytes
//   k_wp_umma      out[128 x 256 tile] = 256 (A_hi B) + (A_lo B): tcgen05.mma kind::i8 (signed x signed for the high bytes,
//                  unsigned x signed for the low bytes), int32 accumulators in TMEM, int64 result written by the epilogue;
//                  split over K with integer atomics (integer addition: any order gives the same words)
// |sum lo w| <= K * 255 * 128 < 2^31 for K <= 65,536 (metal.rs:4234 states the same bound), so int32 never wraps.
#include <cstdlib>

#include "api_internal.h"

using namespace hlapi;

namespace {

constexpr int WP_MT = 128;      // tokens per tile; the stacked tile has 2 * WP_MT rows (hi rows, then lo rows)
constexpr size_t WP_MAX_K = (size_t)1 << 16;

__global__ void __launch_bounds__(256) k_wp_pack(const long long* __restrict__ x, size_t xs, u32 t_rows, u32 K, u32 Kp,
                                                 uint8_t* __restrict__ A /* tiles x 2 x WP_MT x Kp */, int* __restrict__ flag) {
    const u32 t = blockIdx.y;  // padded token index
    const u32 mt = t / WP_MT, r = t % WP_MT;
    uint8_t* hi = A + ((size_t)mt * 2 * WP_MT + r) * Kp;
    uint8_t* lo = hi + (size_t)WP_MT * Kp;
    for (u32 k = blockIdx.x * blockDim.x + threadIdx.x; k < Kp; k += gridDim.x * blockDim.x) {
        long long v = 0;
        if (t < t_rows && k < K) {
            v = x[(size_t)t * xs + k];
            if (v < -32768 || v > 32767) { atomicExch(flag, 1); v = 0; }
        }
        hi[k] = (uint8_t)(v >> 8);
        lo[k] = (uint8_t)(v & 255);
    }
}

// in_out: src[i * N + j] -> dst[j * Kp + i]; else src[j * K + i] -> dst[j * Kp + i]; dst is zero beyond K (memset before)
__global__ void __launch_bounds__(256) k_wp_repack(const int8_t* __restrict__ src, u32 K, u32 N, u32 Kp, int in_out, int8_t* __restrict__ dst) {
    __shared__ int8_t tile[64][65];
    const u32 k0 = blockIdx.x * 64, n0 = blockIdx.y * 64;
    if (in_out) {
        for (u32 e = threadIdx.x; e < 64 * 64; e += blockDim.x) {
            const u32 kk = e / 64, nn = e % 64;  // consecutive threads along n: contiguous in the source
            tile[kk][nn] = (k0 + kk < K && n0 + nn < N) ? src[(size_t)(k0 + kk) * N + n0 + nn] : (int8_t)0;
        }
        __syncthreads();
        for (u32 e = threadIdx.x; e < 64 * 64; e += blockDim.x) {
            const u32 nn = e / 64, kk = e % 64;
            if (n0 + nn < N && k0 + kk < K) dst[(size_t)(n0 + nn) * Kp + k0 + kk] = tile[kk][nn];
        }
    } else {
        for (u32 e = threadIdx.x; e < 64 * 64; e += blockDim.x) {
            const u32 nn = e / 64, kk = e % 64;
            if (n0 + nn < N && k0 + kk < K) dst[(size_t)(n0 + nn) * Kp + k0 + kk] = src[(size_t)(n0 + nn) * K + k0 + kk];
        }
    }
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void mma_s8s8(int (&c)[4], const u32 (&a)[4], const u32 (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// ---------------------------------------------------------------------------------------------------------------
// The product on the 5th-generation tensor cores: tcgen05.mma kind::i8, operands in shared memory, accumulators in TMEM.
// One CTA per SM owns a 128-token tile (two 128-row operands: the signed high bytes and the unsigned low bytes) and 256
// output columns; per K stage of 128 bytes one thread issues 4 x 2 instructions of shape 128 x 256 x 32 (hi: s8 x s8 into
// TMEM columns 0..255, lo: u8 x s8 into columns 256..511), the epilogue reads both accumulators lane by lane and writes
// 256 hi + lo as int64 straight into the result plane (integer atomics when K is split).
// Shared-memory operand layout (K-major, no swizzle): 8-row x 16-byte core matrices of 128 contiguous bytes; the two
// 16-byte K chunks of one instruction are UM_LBO apart, consecutive 8-row groups UM_SBO apart.
// Every wait is bounded: a wait that runs out sets the error word, every thread leaves the loop together and TMEM is freed.
constexpr int UM_NT = 256, UM_KT = 128, UM_STAGES = 3, UM_THREADS = 256;
constexpr u32 UM_LBO = 128, UM_SBO = 1024;
constexpr u32 UM_A_BYTES = WP_MT * UM_KT, UM_B_BYTES = UM_NT * UM_KT, UM_STAGE_BYTES = 2 * UM_A_BYTES + UM_B_BYTES;
constexpr u32 UM_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ u32 um_off(u32 row, u32 chunk) { return (row >> 3) * UM_SBO + chunk * UM_LBO + (row & 7) * 16; }

__device__ __forceinline__ u64 um_desc(u32 smem_addr) {
    // start address, leading and stride byte offsets in 16-byte units; descriptor version 1; layout type 0 (no swizzle)
    return (u64)((smem_addr >> 4) & 0x3FFF) | ((u64)(UM_LBO >> 4) << 16) | ((u64)(UM_SBO >> 4) << 32) | (1ull << 46);
}

// instruction descriptor of kind::i8: D = s32, B = s8, A = s8 or u8, both K-major, N = 256, M = 128
__host__ __device__ constexpr u32 um_idesc(bool a_signed) {
    return (2u << 4) | ((a_signed ? 1u : 0u) << 7) | (1u << 10) | ((u32)(UM_NT >> 3) << 17) | ((u32)(WP_MT >> 4) << 24);
}

__device__ __forceinline__ void um_mma(u32 tmem_d, u64 a_desc, u64 b_desc, u32 idesc, u32 accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void um_commit(u32 mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ bool um_wait(u32 mbar, u32 parity) {
    for (u32 spin = 0; spin < UM_SPIN_LIMIT; spin++) {
        u32 ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(ok)
                     : "r"(mbar), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void um_ld32(u32 taddr, u32 (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
        "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

// grid (N tiles of 256, K splits, token tiles)
__global__ void __launch_bounds__(UM_THREADS, 1) k_wp_umma(const uint8_t* __restrict__ A, const int8_t* __restrict__ B, size_t ldb, u32 N, u32 Kp,
                                                          u32 t_rows, size_t os, long long* __restrict__ out, int* __restrict__ err) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ __align__(8) u64 bars[UM_STAGES + 1];
    __shared__ u32 tmem_slot;
    const u32 tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const u32 n0 = blockIdx.x * UM_NT, mt = blockIdx.z;
    const u32 kt_all = Kp / UM_KT, kt0 = (u32)((u64)kt_all * blockIdx.y / gridDim.y), kt1 = (u32)((u64)kt_all * (blockIdx.y + 1) / gridDim.y);
    const u32 nkt = kt1 - kt0;
    const uint8_t* Ag = A + (size_t)mt * 2 * WP_MT * Kp;
    const u32 smem_base = (u32)__cvta_generic_to_shared(smem);
    const u32 bar_base = (u32)__cvta_generic_to_shared(bars);

    if (tid == 0) {
        for (int i = 0; i <= UM_STAGES; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_base + 8 * i));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::);
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"((u32)__cvta_generic_to_shared(&tmem_slot)), "r"(512u));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::);
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
    const u32 tmem = tmem_slot;

    auto load_stage = [&](u32 kt, u32 st) {
        const u32 k0 = kt * UM_KT;
        uint8_t* sa = smem + (size_t)st * UM_STAGE_BYTES;
        uint8_t* sb = sa + 2 * UM_A_BYTES;
#pragma unroll
        for (int i = 0; i < 2 * WP_MT * 8 / UM_THREADS; i++) {  // stacked rows: 0..127 the high bytes, 128..255 the low bytes
            const u32 e = tid + i * UM_THREADS, row = e >> 3, c = e & 7;
            cp_async16(sa + (row >> 7) * UM_A_BYTES + um_off(row & 127, c), Ag + (size_t)row * Kp + k0 + c * 16);
        }
#pragma unroll
        for (int i = 0; i < UM_NT * 8 / UM_THREADS; i++) {
            const u32 e = tid + i * UM_THREADS, row = e >> 3, c = e & 7;
            const u32 n = min(n0 + row, N - 1);  // columns past N repeat the last one; they are never written out
            cp_async16(sb + um_off(row, c), B + (size_t)n * ldb + k0 + c * 16);
        }
    };

#pragma unroll
    for (int s = 0; s < UM_STAGES - 1; s++) {
        if ((u32)s < nkt) load_stage(kt0 + s, s);
        cp_async_commit();
    }
    bool failed = false;
    for (u32 it = 0; it < nkt; it++) {
        cp_async_wait<UM_STAGES - 2>();
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the copies above are generic-proxy writes; the tensor core reads through the async proxy
        __syncthreads();
        const u32 st = it % UM_STAGES;
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
            const u32 sa = smem_base + st * UM_STAGE_BYTES, sb = sa + 2 * UM_A_BYTES;
#pragma unroll
            for (u32 kk = 0; kk < UM_KT / 32; kk++) {
                const u64 bd = um_desc(sb + kk * 2 * UM_LBO);
                const u32 accumulate = (it | kk) ? 1u : 0u;
                um_mma(tmem, um_desc(sa + kk * 2 * UM_LBO), bd, um_idesc(true), accumulate);
                um_mma(tmem + 256, um_desc(sa + UM_A_BYTES + kk * 2 * UM_LBO), bd, um_idesc(false), accumulate);
            }
            um_commit(bar_base + 8 * st);  // arrives when the instructions above have read this stage
        }
        // the stage the next copies overwrite was read by the instructions issued one iteration ago
        bool ok = true;
        if (it >= 1 && it + UM_STAGES - 1 < nkt) ok = um_wait(bar_base + 8 * ((it - 1) % UM_STAGES), ((it - 1) / UM_STAGES) & 1);
        failed = __syncthreads_or(!ok);
        if (failed) break;
        if (it + UM_STAGES - 1 < nkt) load_stage(kt0 + it + UM_STAGES - 1, (it + UM_STAGES - 1) % UM_STAGES);
        cp_async_commit();
    }
    cp_async_wait<0>();
    if (!failed) {
        if (tid == 0) um_commit(bar_base + 8 * UM_STAGES);  // arrives when every instruction of this CTA has completed
        const bool ok = um_wait(bar_base + 8 * UM_STAGES, 0);
        failed = __syncthreads_or(!ok);
    }
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
    if (!failed && nkt) {
        // warp w reads TMEM lanes 32 (w % 4) .. +31 (the rows of the token tile), columns 128 (w / 4) .. +127
        const u32 q = warp & 3, half = warp >> 2;
        const u32 row = q * 32 + lane, t = mt * WP_MT + row;
        const bool split = gridDim.y > 1;
#pragma unroll 1
        for (u32 cc = 0; cc < 4; cc++) {
            const u32 col = half * 128 + cc * 32;
            u32 hi[32], lo[32];
            um_ld32(tmem + ((q * 32) << 16) + col, hi);
            um_ld32(tmem + ((q * 32) << 16) + 256 + col, lo);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            if (t < t_rows) {
                long long* o = out + (size_t)t * os + n0 + col;
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    if (n0 + col + j < N) {
                        const long long v = 256ll * (int)hi[j] + (int)lo[j];
                        if (split) atomicAdd(reinterpret_cast<unsigned long long*>(o + j), (unsigned long long)v);
                        else o[j] = v;
                    }
                }
            }
        }
    }
    if (failed && tid == 0) atomicExch(err, 2);
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::);
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512u));
}

// Register-resident int8 tensor-core products: the ceiling of the m16n8k32 instruction the product kernel issues (16
// independent accumulators per warp, 8 warps per CTA, 2 CTAs per SM, operands never reloaded).
__global__ void __launch_bounds__(256, 2) k_mma_i8_peak(u32 iters, int* __restrict__ sink) {
    int acc[4][4][4];
    u32 a[4][4], b[4][2];
#pragma unroll
    for (int m = 0; m < 4; m++)
#pragma unroll
        for (int i = 0; i < 4; i++) a[m][i] = threadIdx.x * 0x01010101u + 16 * m + i;
#pragma unroll
    for (int n = 0; n < 4; n++) {
        b[n][0] = threadIdx.x ^ (0x7F3C11A5u + n);
        b[n][1] = blockIdx.x + 0x01020304u * (n + 1);
    }
#pragma unroll
    for (int m = 0; m < 4; m++)
#pragma unroll
        for (int n = 0; n < 4; n++)
#pragma unroll
            for (int x = 0; x < 4; x++) acc[m][n][x] = 0;
    // the product kernel's own register pattern: 4 A tiles x 4 B tiles, 16 accumulators
    for (u32 it = 0; it < iters; it++) {
#pragma unroll
        for (int m = 0; m < 4; m++)
#pragma unroll
            for (int n = 0; n < 4; n++) mma_s8s8(acc[m][n], a[m], b[n]);
    }
    int v = 0;
#pragma unroll
    for (int m = 0; m < 4; m++)
#pragma unroll
        for (int n = 0; n < 4; n++) v ^= acc[m][n][0] ^ acc[m][n][3];
    if (v == 0x5EED5EED) sink[0] = v;
}

// everything on the context's stream; d_* are device pointers; *flag_out is read after one synchronisation
int product_on_device(hl_ctx* c, size_t t_rows, const int64_t* d_x, size_t xs, const int8_t* d_w, size_t K, size_t N, size_t os, size_t out_len,
                      int in_out, int64_t* d_out, int* taken) {
    const u32 Kp = (u32)((K + UM_KT - 1) / UM_KT * UM_KT);
    const u32 tiles = (u32)((t_rows + WP_MT - 1) / WP_MT);
    const bool in_place = !in_out && K % UM_KT == 0 && ((uintptr_t)d_w & 15) == 0;
    const size_t a_bytes = (size_t)tiles * 2 * WP_MT * Kp, b_bytes = in_place ? 0 : (size_t)N * Kp;
    uint8_t* d_a = nullptr;
    int8_t* d_b = nullptr;
    int* d_flag = nullptr;
    int rc = dev_alloc(c, (void**)&d_a, a_bytes);
    if (!rc) rc = dev_alloc(c, (void**)&d_flag, 4);
    if (!rc && b_bytes) rc = dev_alloc(c, (void**)&d_b, b_bytes);
    // every CTA does the same work, so what counts is how full the last wave of one CTA per SM is: the smallest split over K
    // that fills the waves best; each further split adds a pass of integer atomics over the plane, charged at 3 %
    const u32 n_tiles = (u32)((N + UM_NT - 1) / UM_NT), kt_all = Kp / UM_KT;
    const u32 slots = (u32)c->sm_count, base = n_tiles * tiles;
    u32 splits = 1;
    double best = 0.0;
    for (u32 sp = 1; sp <= 32 && sp <= kt_all; sp++) {
        const u64 ctas = (u64)base * sp;
        const double eff = (double)ctas / (double)((ctas + slots - 1) / slots * slots) / (1.0 + 0.03 * (sp - 1));
        if (eff > best + 0.02) { best = eff; splits = sp; }
    }
    // HL_B200_WP_SPLITS=<n>: a tuning override of the split (the result does not depend on it)
    if (const char* ov = getenv("HL_B200_WP_SPLITS")) {
        const long v = atol(ov);
        if (v >= 1 && v <= (long)kt_all && v <= 65535) splits = (u32)v;
    }
    int flag = 0;
    if (!rc) {
        Timed t(c, HL_T_WITNESS);
        cudaError_t e = cudaMemsetAsync(d_flag, 0, 4, c->stream);
        if (e == cudaSuccess) e = cudaMemsetAsync(d_out, 0, out_len * 8, c->stream);
        if (e == cudaSuccess && b_bytes) e = cudaMemsetAsync(d_b, 0, b_bytes, c->stream);
        if (e == cudaSuccess) {
            k_wp_pack<<<dim3((Kp + 1023) / 1024, tiles * WP_MT), 256, 0, c->stream>>>((const long long*)d_x, xs, (u32)t_rows, (u32)K, Kp, d_a, d_flag);
            e = cudaGetLastError();
            c->stats.kernel_launches++;
        }
        if (e == cudaSuccess && b_bytes) {
            k_wp_repack<<<dim3(Kp / 64, (unsigned)((N + 63) / 64)), 256, 0, c->stream>>>(d_w, (u32)K, (u32)N, Kp, in_out, d_b);
            e = cudaGetLastError();
            c->stats.kernel_launches++;
        }
        const size_t smem = (size_t)UM_STAGES * UM_STAGE_BYTES;
        if (e == cudaSuccess) e = cudaFuncSetAttribute(k_wp_umma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) {
            k_wp_umma<<<dim3(n_tiles, splits, tiles), UM_THREADS, smem, c->stream>>>(d_a, in_place ? d_w : d_b, in_place ? K : (size_t)Kp, (u32)N, Kp,
                                                                                   (u32)t_rows, os, (long long*)d_out, d_flag);
            e = cudaGetLastError();
            c->stats.kernel_launches++;
        }
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "witness product launch", e);
    }
    if (!rc) rc = d2h(c, &flag, d_flag, 4);
    if (!rc) rc = sync(c, "witness_product");
    else cudaStreamSynchronize(c->stream);
    if (d_a) dev_free(c, d_a, a_bytes);
    if (d_flag) dev_free(c, d_flag, 4);
    if (d_b) dev_free(c, d_b, b_bytes);
    if (!rc && flag == 2) rc = fail(c, HL_B200_ERR_TIMEOUT, "witness product: a bounded wait on the tensor-core pipeline ran out");
    if (!rc) *taken = flag ? 0 : 1;
    return rc;
}

// witness_product_with's `fits` (metal.rs:4662-4674)
bool shape_fits(size_t t_rows, size_t x_len, size_t xs, size_t w_len, size_t inner, size_t outer, size_t os, size_t out_len) {
    // the reference's bounds are 2^30 rows and columns; the grids here take 2^15 rows and 2^21 columns
    if (t_rows < 1 || inner < 1 || outer < 1 || inner > WP_MAX_K || t_rows > ((size_t)1 << 15) || outer > ((size_t)1 << 21)) return false;
    if (xs < inner || os < outer || os > 0xFFFFFFFFull) return false;
    if (xs > ((size_t)1 << 40) || (t_rows - 1) * xs + inner > x_len) return false;
    if ((t_rows - 1) * os + outer > out_len) return false;
    return inner * outer <= w_len;
}

}  // namespace

extern "C" {

int hl_b200_mma_i8_peak(hl_ctx* c, uint32_t iters, double* macs_per_second) {
    if (!c || !macs_per_second || iters == 0) return fail(c, HL_B200_ERR_ARG, "mma_i8_peak: argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    int* d_sink = nullptr;
    int rc = dev_alloc(c, (void**)&d_sink, 4);
    cudaEvent_t a = nullptr, b = nullptr;
    float ms = 0.f;
    const int blocks = c->sm_count * 2;
    if (!rc) {
        cudaEventCreate(&a); cudaEventCreate(&b);
        k_mma_i8_peak<<<blocks, 256, 0, c->stream>>>(8, d_sink);  // warm-up
        cudaEventRecord(a, c->stream);
        k_mma_i8_peak<<<blocks, 256, 0, c->stream>>>(iters, d_sink);
        cudaEventRecord(b, c->stream);
        c->stats.kernel_launches += 2;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "mma_i8_peak launch", e);
    }
    if (!rc) rc = sync(c, "mma_i8_peak");
    if (!rc && cudaEventElapsedTime(&ms, a, b) != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "mma_i8_peak timing");
    if (a) cudaEventDestroy(a);
    if (b) cudaEventDestroy(b);
    if (d_sink) dev_free(c, d_sink, 4);
    if (!rc) *macs_per_second = (double)blocks * 8 * 16.0 * 4096.0 * iters / (ms * 1e-3);
    return rc;
}

int hl_b200_witness_product_dev(hl_ctx* c, size_t t_rows, const int64_t* d_x, size_t x_len, size_t xs, const int8_t* d_w, size_t w_len, size_t inner,
                                size_t outer, size_t os, size_t out_len, int in_out, int64_t* d_out, int* taken) {
    if (!c || !taken) return fail(c, HL_B200_ERR_ARG, "witness_product: null argument");
    *taken = 0;
    if (!shape_fits(t_rows, x_len, xs, w_len, inner, outer, os, out_len)) return HL_B200_OK;
    if (!d_x || !d_w || !d_out) return fail(c, HL_B200_ERR_ARG, "witness_product: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    return product_on_device(c, t_rows, d_x, xs, d_w, inner, outer, os, out_len, in_out, d_out, taken);
}

int hl_b200_witness_product(hl_ctx* c, size_t t_rows, const int64_t* x, size_t x_len, size_t xs, const int8_t* w, size_t w_len, size_t inner,
                            size_t outer, size_t os, size_t out_len, int in_out, int64_t* out, int* taken) {
    if (!c || !taken) return fail(c, HL_B200_ERR_ARG, "witness_product: null argument");
    *taken = 0;
    if (!shape_fits(t_rows, x_len, xs, w_len, inner, outer, os, out_len)) return HL_B200_OK;
    if (!x || !w || !out) return fail(c, HL_B200_ERR_ARG, "witness_product: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    const size_t xb = ((t_rows - 1) * xs + inner) * 8, wb = inner * outer, ob = out_len * 8;
    int64_t *d_x = nullptr, *d_out = nullptr;
    int8_t* d_w = nullptr;
    int rc = dev_alloc(c, (void**)&d_x, xb);
    if (!rc) rc = dev_alloc(c, (void**)&d_w, wb);
    if (!rc) rc = dev_alloc(c, (void**)&d_out, ob);
    if (!rc) rc = h2d(c, d_x, x, xb);
    if (!rc) rc = h2d(c, d_w, w, wb);
    if (!rc) rc = product_on_device(c, t_rows, d_x, xs, d_w, inner, outer, os, out_len, in_out, d_out, taken);
    if (!rc && *taken) rc = d2h(c, out, d_out, ob);
    if (!rc) rc = sync(c, "witness_product");
    else cudaStreamSynchronize(c->stream);
    if (d_x) dev_free(c, d_x, xb);
    if (d_w) dev_free(c, d_w, wb);
    if (d_out) dev_free(c, d_out, ob);
    return rc;
}

}  // extern "C"
