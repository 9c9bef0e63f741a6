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
#include <cuda.h>

#include <cstdlib>

#include "api_internal.h"

using namespace hlapi;

namespace {

constexpr int WP_MT = 128;      // tokens per tile; the stacked tile has 2 * WP_MT rows (hi rows, then lo rows)
constexpr size_t WP_MAX_K = (size_t)1 << 16;

__global__ void __launch_bounds__(256) k_wp_pack(const long long* __restrict__ x, size_t xs, u32 t_rows, u32 K, u32 Kp,
                                                 uint8_t* __restrict__ A /* tiles x 2 x WP_MT x Kp */, int* __restrict__ flag,
                                                 long long* __restrict__ clear, size_t clear_words) {
    // the result plane's clear rides along (the product kernel runs after this one): one launch less on a launch-bound path
    for (size_t i = ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x; i < clear_words;
         i += (size_t)gridDim.x * gridDim.y * blockDim.x)
        clear[i] = 0;
    const u32 t = blockIdx.y;  // padded token index
    const u32 mt = t / WP_MT, r = t % WP_MT;
    uint8_t* hi = A + ((size_t)mt * 2 * WP_MT + r) * Kp;
    uint8_t* lo = hi + (size_t)WP_MT * Kp;
    // four activations (one 32-byte sector) per thread, one 4-byte word of each plane out
    for (u32 k = (blockIdx.x * blockDim.x + threadIdx.x) * 4; k < Kp; k += gridDim.x * blockDim.x * 4) {
        u32 h = 0, l = 0;
        bool bad = false;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            long long v = 0;
            if (t < t_rows && k + j < K) {
                v = x[(size_t)t * xs + k + j];
                if (v < -32768 || v > 32767) { bad = true; v = 0; }
            }
            h |= (u32)((v >> 8) & 255) << (8 * j);
            l |= (u32)(v & 255) << (8 * j);
        }
        if (bad) atomicExch(flag, 1);
        *reinterpret_cast<u32*>(hi + k) = h;
        *reinterpret_cast<u32*>(lo + k) = l;
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

// ---------------------------------------------------------------------------------------------------------------
// The product on the 5th-generation tensor cores: TMA tiles into shared memory, tcgen05.mma kind::i8, accumulators in TMEM.
// One CTA per SM owns a 128-token tile (two 128-row operands: the signed high bytes and the unsigned low bytes) and 256
// output columns.  Per K stage of 128 bytes one thread asks the TMA unit for two boxes (256 stacked activation rows and 256
// weight rows of 128 bytes, 128-byte swizzle) and, when they have landed, issues 4 x 2 instructions of shape 128 x 256 x 32
// (hi: s8 x s8 into TMEM columns 0..255, lo: u8 x s8 into columns 256..511); the epilogue reads both accumulators lane by
// lane and writes 256 hi + lo as int64 straight into the result plane (integer atomics when K is split).
// Shared-memory operands are K-major with the 128-byte swizzle the TMA unit writes: rows of 128 bytes, 8-row groups
// UM_SBO apart, a K step of 32 bytes is 32 bytes further along the row.
// Every wait is bounded: a wait that runs out sets the error word, every thread leaves together and TMEM is freed.
constexpr int UM_NT = 256, UM_KT = 128, UM_STAGES = 3, UM_THREADS = 256;
constexpr u32 UM_SBO = 1024;
constexpr u32 UM_A_BYTES = WP_MT * UM_KT, UM_B_BYTES = UM_NT * UM_KT, UM_STAGE_BYTES = 2 * UM_A_BYTES + UM_B_BYTES;
constexpr u32 UM_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ u64 um_desc(u32 smem_addr) {
    // start address and stride byte offset in 16-byte units (the leading offset is not used by a swizzled K-major operand and is
    // set to 1 as the canonical form has it); descriptor version 1; layout type 2 = 128-byte swizzle
    return (u64)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | ((u64)(UM_SBO >> 4) << 32) | (1ull << 46) | (2ull << 61);
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
// one box of the tensor map into shared memory; its bytes are counted on the mbarrier
__device__ __forceinline__ void um_tma_2d(u32 smem_dst, const CUtensorMap* map, u32 mbar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(smem_dst),
                 "l"((u64)map), "r"(mbar), "r"(x), "r"(y)
                 : "memory");
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

// grid (N tiles of 256, K splits, token tiles).  map_a: the packed activations, (tiles * 256) rows of Kp bytes; map_b: the weights,
// N rows of K bytes (rows past N read as zero).  Barriers: full[s] (the stage's two boxes have landed), empty[s] (the instructions
// that read the stage have completed), done.
__global__ void __launch_bounds__(UM_THREADS, 1) k_wp_umma(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, u32 N,
                                                          u32 Kp, u32 t_rows, size_t os, long long* __restrict__ out, int* __restrict__ err) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ __align__(8) u64 bars[2 * UM_STAGES + 1];
    __shared__ u32 tmem_slot;
    __shared__ volatile u32 gave_up;  // set by the issuing thread when one of its waits ran out
    const u32 tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const u32 n0 = blockIdx.x * UM_NT, mt = blockIdx.z;
    const u32 kt_all = Kp / UM_KT, kt0 = (u32)((u64)kt_all * blockIdx.y / gridDim.y), kt1 = (u32)((u64)kt_all * (blockIdx.y + 1) / gridDim.y);
    const u32 nkt = kt1 - kt0;
    const u32 smem_base = ((u32)__cvta_generic_to_shared(smem_raw) + 1023u) & ~1023u;  // the swizzle pattern repeats every 1024 bytes
    const u32 bar_base = (u32)__cvta_generic_to_shared(bars);
    const u32 full0 = bar_base, empty0 = bar_base + 8 * UM_STAGES, done = bar_base + 16 * UM_STAGES;

    if (tid == 0) {
        gave_up = 0;
        for (int i = 0; i <= 2 * UM_STAGES; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_base + 8 * i));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::);
    }
    if (warp == 0) {
        // all 512 columns: the allocation cannot wait on another CTA, because this kernel's shared memory (3 stages of 64 KB) lets
        // only one CTA live on an SM and no other kernel of the library holds TMEM
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"((u32)__cvta_generic_to_shared(&tmem_slot)), "r"(512u));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::);
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
    const u32 tmem = tmem_slot;

    bool ok = true;
    if (tid == 0) {
        auto load_stage = [&](u32 kt, u32 st) {
            const u32 sa = smem_base + st * UM_STAGE_BYTES;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(full0 + 8 * st), "r"(UM_STAGE_BYTES) : "memory");
            um_tma_2d(sa, &map_a, full0 + 8 * st, (int)(kt * UM_KT), (int)(mt * 2 * WP_MT));
            um_tma_2d(sa + 2 * UM_A_BYTES, &map_b, full0 + 8 * st, (int)(kt * UM_KT), (int)n0);
        };
        for (u32 s = 0; s < UM_STAGES && s < nkt; s++) load_stage(kt0 + s, s);
        for (u32 it = 0; it < nkt && ok; it++) {
            const u32 st = it % UM_STAGES;
            ok = um_wait(full0 + 8 * st, (it / UM_STAGES) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
            const u32 sa = smem_base + st * UM_STAGE_BYTES, sb = sa + 2 * UM_A_BYTES;
#pragma unroll
            for (u32 kk = 0; kk < UM_KT / 32; kk++) {
                const u64 bd = um_desc(sb + kk * 32);
                const u32 accumulate = (it | kk) ? 1u : 0u;
                um_mma(tmem, um_desc(sa + kk * 32), bd, um_idesc(true), accumulate);
                um_mma(tmem + 256, um_desc(sa + UM_A_BYTES + kk * 32), bd, um_idesc(false), accumulate);
            }
            um_commit(empty0 + 8 * st);  // arrives when the instructions above have read this stage
            // refill the stage read one iteration ago, once its instructions have completed
            if (it >= 1 && it - 1 + UM_STAGES < nkt) {
                ok = um_wait(empty0 + 8 * ((it - 1) % UM_STAGES), ((it - 1) / UM_STAGES) & 1);
                if (ok) load_stage(kt0 + it - 1 + UM_STAGES, (it - 1) % UM_STAGES);
            }
        }
        if (ok) um_commit(done);  // arrives when every instruction of this CTA has completed
        else gave_up = 1;
    }
    // everyone waits for the accumulators, in slices so that a wait the issuing thread gave up on ends the others' too
    bool ready = false;
    for (u32 round = 0; round < 1024 && !ready && !gave_up; round++) {
        for (u32 spin = 0; spin < (UM_SPIN_LIMIT >> 10) && !ready; spin++) {
            u32 p;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                         : "=r"(p)
                         : "r"(done), "r"(0u)
                         : "memory");
            ready = p != 0;
            if (!ready) __nanosleep(128);  // the polling threads stay off the shared memory the tensor core is reading
        }
    }
    const bool failed = __syncthreads_or(!ready);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
    if (!failed) {
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

// everything on the context's stream; d_* are device pointers; *flag_out is read after one synchronisation
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// a byte matrix of `rows` rows of `inner` readable bytes, `pitch` bytes apart (a multiple of 16), read in boxes of 128 bytes x 256 rows
// with the 128-byte swizzle; rows and bytes outside the matrix read as zero
int byte_matrix_map(hl_ctx* c, const void* base, size_t inner, size_t rows, size_t pitch, CUtensorMap* map) {
    // looked up once per process (a function-local static is initialised under the language's own lock)
    static const EncodeTiledFn encode = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) fn = nullptr;
        return (EncodeTiledFn)fn;
    }();
    if (!encode) return fail(c, HL_B200_ERR_DEVICE, "witness product: the driver has no tensor-map encoder");
    const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows}, strides[1] = {(cuuint64_t)pitch};
    const cuuint32_t box[2] = {(cuuint32_t)UM_KT, 256u}, elem[2] = {1u, 1u};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? HL_B200_OK : fail(c, HL_B200_ERR_DEVICE, "witness product: tensor-map encoding refused");
}

int product_on_device(hl_ctx* c, size_t t_rows, const int64_t* d_x, size_t xs, const int8_t* d_w, size_t K, size_t N, size_t os, size_t out_len,
                      int in_out, int64_t* d_out, int* taken) {
    const u32 Kp = (u32)((K + UM_KT - 1) / UM_KT * UM_KT);
    const u32 tiles = (u32)((t_rows + WP_MT - 1) / WP_MT);
    // weights are read in place when their rows are whole K stages and there is at least one box of rows; else from a padded copy
    const bool in_place = !in_out && K % UM_KT == 0 && ((uintptr_t)d_w & 15) == 0 && N >= (size_t)UM_NT;
    const size_t n_pad = (N + UM_NT - 1) / UM_NT * UM_NT;
    const size_t a_bytes = (size_t)tiles * 2 * WP_MT * Kp, b_bytes = in_place ? 0 : n_pad * Kp;
    uint8_t* d_a = nullptr;
    int8_t* d_b = nullptr;
    int rc = dev_alloc(c, (void**)&d_a, a_bytes);
    if (!rc && !c->d_wp_flag) {  // the status word lives with the context and is zero between calls: no clear on the launch path
        if (cudaMalloc((void**)&c->d_wp_flag, 4) != cudaSuccess || cudaMemsetAsync(c->d_wp_flag, 0, 4, c->stream) != cudaSuccess) {
            c->d_wp_flag = nullptr;
            rc = fail(c, HL_B200_ERR_OOM, "witness product: status word");
        }
    }
    int* d_flag = c->d_wp_flag;
    if (!rc && b_bytes) rc = dev_alloc(c, (void**)&d_b, b_bytes);
    CUtensorMap map_a, map_b;
    if (!rc) rc = byte_matrix_map(c, d_a, Kp, (size_t)tiles * 2 * WP_MT, Kp, &map_a);
    if (!rc) rc = byte_matrix_map(c, in_place ? (const void*)d_w : (const void*)d_b, Kp, in_place ? N : n_pad, Kp, &map_b);
    // The split over K by a cost model fitted to measurements on B200: a CTA streams one K stage (64 KB of operands) in about
    // 1.3 us, CTAs run in waves of one per SM, and every split beyond the first adds a pass of 64-bit integer atomics over the
    // result plane at about 195 G atomics per second.
    const u32 n_tiles = (u32)((N + UM_NT - 1) / UM_NT), kt_all = Kp / UM_KT;
    const u32 slots = (u32)c->sm_count, base = n_tiles * tiles;
    u32 splits = 1;
    double best = 1e30;
    for (u32 sp = 1; sp <= 64 && sp <= kt_all; sp++) {
        const u64 ctas = (u64)base * sp;
        const double waves = (double)((ctas + slots - 1) / slots), stages = (double)((kt_all + sp - 1) / sp);
        const double cost = waves * stages * 1.3e-6 + (sp > 1 ? (double)sp * (double)tiles * WP_MT * (double)N / 195e9 : 0.0);
        if (cost < best * 0.98) { best = cost; splits = sp; }
    }
    int flag = 0;
    if (!rc) {
        Timed t(c, HL_T_WITNESS);
        // the plane is cleared unless the product kernel writes every word of it exactly once
        const bool dense = splits == 1 && os == N && out_len == t_rows * N;
        cudaError_t e = cudaSuccess;
        if (e == cudaSuccess && b_bytes) e = cudaMemsetAsync(d_b, 0, b_bytes, c->stream);
        if (e == cudaSuccess) {
            k_wp_pack<<<dim3((Kp + 1023) / 1024, tiles * WP_MT), 256, 0, c->stream>>>((const long long*)d_x, xs, (u32)t_rows, (u32)K, Kp, d_a, d_flag,
                                                                                       (long long*)d_out, dense ? 0 : out_len);
            e = cudaGetLastError();
            c->stats.kernel_launches++;
        }
        if (e == cudaSuccess && b_bytes) {
            k_wp_repack<<<dim3(Kp / 64, (unsigned)((N + 63) / 64)), 256, 0, c->stream>>>(d_w, (u32)K, (u32)N, Kp, in_out, d_b);
            e = cudaGetLastError();
            c->stats.kernel_launches++;
        }
        const size_t smem = (size_t)UM_STAGES * UM_STAGE_BYTES + 1024;
        if (e == cudaSuccess && !c->wp_attr) {
            e = cudaFuncSetAttribute(k_wp_umma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            c->wp_attr = e == cudaSuccess;
        }
        if (e == cudaSuccess) {
            k_wp_umma<<<dim3(n_tiles, splits, tiles), UM_THREADS, smem, c->stream>>>(map_a, map_b, (u32)N, Kp, (u32)t_rows, os, (long long*)d_out, d_flag);
            e = cudaGetLastError();
            c->stats.kernel_launches++;
        }
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "witness product launch", e);
    }
    if (!rc) rc = d2h(c, &flag, d_flag, 4);
    if (!rc) rc = sync(c, "witness_product");
    else cudaStreamSynchronize(c->stream);
    if (flag && d_flag) cudaMemsetAsync(d_flag, 0, 4, c->stream);  // back to zero for the next call
    if (d_a) dev_free(c, d_a, a_bytes);
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
