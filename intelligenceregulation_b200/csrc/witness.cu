// Witness weight products (hashline/src/gpu/metal.rs:4646-4680 witness_product; private_block/witness.rs:979-991): the one
// dense contraction of the system, exact integers: int16 activations times int8 weights into int64.
//
//   k_wp_pack      x (int64, row stride xs) -> two byte planes per 128-token tile: hi = x >> 8 (signed), lo = x & 255
//                  (unsigned), K padded with zeros to a multiple of 64; an activation outside int16 raises the flag
//   k_wp_repack    weights the product kernel cannot read in place (in_out layout, or K not a multiple of 64) -> rows of Kp bytes
//   k_wp_gemm      P[256 x N] += A[256 x K] B[K x N] per 128-token tile, int8 tensor-core products (m16n8k32: signed x signed
//                  for the hi rows, unsigned x signed for the lo rows), int32 accumulators, split over K with integer atomics
//                  (integer addition: any order gives the same words)
//   k_wp_combine   out[t * os + j] = 256 P_hi[t][j] + P_lo[t][j] in int64
// |sum lo w| <= K * 255 * 128 < 2^31 for K <= 65,536 (metal.rs:4234 states the same bound), so int32 never wraps.
#include "api_internal.h"

using namespace hlapi;

namespace {

constexpr int WP_MT = 128;      // tokens per tile; the stacked tile has 2 * WP_MT rows (hi rows, then lo rows)
constexpr int WP_NT = 128;      // output columns per CTA
constexpr int WP_KT = 128;      // K bytes per stage: whole 128-byte lines of every row
constexpr int WP_LD = WP_KT + 16;  // shared-memory row pitch in bytes: 36 words, so the 8 rows of a fragment fall in distinct banks
constexpr int WP_STAGES = 3;
constexpr int WP_THREADS = 512;  // 16 warps: 4 over the stacked rows x 4 over the columns, 64 x 32 outputs each
constexpr int WP_CTAS_PER_SM = 1;
constexpr int WP_CH = WP_KT / 16;  // 16-byte chunks per row and stage
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

// four 8 x 16-byte matrices from shared memory, one row address per lane (lanes 8 i .. 8 i + 7 give matrix i)
__device__ __forceinline__ void ldmatrix_x4(u32 (&r)[4], const void* smem_row) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

__device__ __forceinline__ void mma_s8s8(int (&c)[4], const u32 (&a)[4], const u32 (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], const u32 (&a)[4], const u32 (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// grid (N tiles, K splits, token tiles); B rows of ldb bytes hold one output column's K weights, readable up to Kp
__global__ void __launch_bounds__(WP_THREADS, WP_CTAS_PER_SM) k_wp_gemm(const uint8_t* __restrict__ A, const int8_t* __restrict__ B, size_t ldb, u32 N, u32 Kp,
                                                          u32 Np, int* __restrict__ P /* tiles x 2 WP_MT x Np */) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* As = smem;                                        // stages x 256 x WP_LD
    uint8_t* Bs = smem + (size_t)WP_STAGES * 2 * WP_MT * WP_LD;  // stages x WP_NT x WP_LD
    const u32 tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const u32 warp_m = warp & 3, warp_n = warp >> 2;
    const u32 n0 = blockIdx.x * WP_NT, mt = blockIdx.z;
    const u32 kt_all = Kp / WP_KT, kt0 = (u32)((u64)kt_all * blockIdx.y / gridDim.y), kt1 = (u32)((u64)kt_all * (blockIdx.y + 1) / gridDim.y);
    const uint8_t* Ag = A + (size_t)mt * 2 * WP_MT * Kp;

    auto load_stage = [&](u32 kt, u32 st) {
        const u32 k0 = kt * WP_KT;
        uint8_t* as = As + (size_t)st * 2 * WP_MT * WP_LD;
        uint8_t* bs = Bs + (size_t)st * WP_NT * WP_LD;
#pragma unroll
        for (int i = 0; i < 2 * WP_MT * WP_CH / WP_THREADS; i++) {
            const u32 e = tid + i * WP_THREADS, row = e / WP_CH, c = e % WP_CH;
            cp_async16(as + row * WP_LD + c * 16, Ag + (size_t)row * Kp + k0 + c * 16);
        }
#pragma unroll
        for (int i = 0; i < WP_NT * WP_CH / WP_THREADS; i++) {
            const u32 e = tid + i * WP_THREADS, row = e / WP_CH, c = e % WP_CH;
            const u32 n = min(n0 + row, N - 1);  // columns past N repeat the last one; they are never written out
            cp_async16(bs + row * WP_LD + c * 16, B + (size_t)n * ldb + k0 + c * 16);
        }
    };

    int acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int x = 0; x < 4; x++) acc[i][j][x] = 0;

    const u32 nkt = kt1 - kt0;
#pragma unroll
    for (int s = 0; s < WP_STAGES - 1; s++) {
        if ((u32)s < nkt) load_stage(kt0 + s, s);
        cp_async_commit();
    }
    for (u32 it = 0; it < nkt; it++) {
        cp_async_wait<WP_STAGES - 2>();
        __syncthreads();  // stage `it` has landed for every thread, and stage it-1's readers are done
        if (it + WP_STAGES - 1 < nkt) load_stage(kt0 + it + WP_STAGES - 1, (it + WP_STAGES - 1) % WP_STAGES);
        cp_async_commit();
        const uint8_t* as = As + (size_t)(it % WP_STAGES) * 2 * WP_MT * WP_LD + (size_t)(warp_m * 64) * WP_LD;
        const uint8_t* bs = Bs + (size_t)(it % WP_STAGES) * WP_NT * WP_LD + (size_t)(warp_n * 32) * WP_LD;
#pragma unroll
        for (int kk = 0; kk < WP_KT; kk += 32) {
            // fragments of m16n8k32 with 8-bit operands: A = (rows g / g + 8) x (bytes 4 tig.. / 16 + 4 tig..), B = column g x the same
            // bytes: exactly the 8 x 16-byte matrices ldmatrix hands out, one instruction per A tile and per pair of B tiles
            u32 a[4][4], b[4][2];
#pragma unroll
            for (int mi = 0; mi < 4; mi++)
                ldmatrix_x4(a[mi], as + (size_t)(mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * WP_LD + kk + (lane >> 4) * 16);
#pragma unroll
            for (int np = 0; np < 2; np++) {
                u32 r[4];
                ldmatrix_x4(r, bs + (size_t)(np * 16 + (lane & 7) + (lane >> 4) * 8) * WP_LD + kk + ((lane >> 3) & 1) * 16);
                b[2 * np][0] = r[0]; b[2 * np][1] = r[1]; b[2 * np + 1][0] = r[2]; b[2 * np + 1][1] = r[3];
            }
            if (warp_m < 2) {  // rows 0..127 of the stacked tile: the signed high bytes
#pragma unroll
                for (int mi = 0; mi < 4; mi++)
#pragma unroll
                    for (int ni = 0; ni < 4; ni++) mma_s8s8(acc[mi][ni], a[mi], b[ni]);
            } else {            // rows 128..255: the unsigned low bytes
#pragma unroll
                for (int mi = 0; mi < 4; mi++)
#pragma unroll
                    for (int ni = 0; ni < 4; ni++) mma_u8s8(acc[mi][ni], a[mi], b[ni]);
            }
        }
    }
    cp_async_wait<0>();
    int* Pt = P + (size_t)mt * 2 * WP_MT * Np;
    const bool split = gridDim.y > 1;
#pragma unroll
    for (int mi = 0; mi < 4; mi++)
#pragma unroll
        for (int ni = 0; ni < 4; ni++) {
            const u32 row = warp_m * 64 + mi * 16 + g, col = n0 + warp_n * 32 + ni * 8 + tig * 2;
            int* p0 = Pt + (size_t)row * Np + col;
            int* p1 = p0 + (size_t)8 * Np;
            if (split) {
                atomicAdd(p0, acc[mi][ni][0]); atomicAdd(p0 + 1, acc[mi][ni][1]);
                atomicAdd(p1, acc[mi][ni][2]); atomicAdd(p1 + 1, acc[mi][ni][3]);
            } else {
                *reinterpret_cast<int2*>(p0) = make_int2(acc[mi][ni][0], acc[mi][ni][1]);
                *reinterpret_cast<int2*>(p1) = make_int2(acc[mi][ni][2], acc[mi][ni][3]);
            }
        }
}

__global__ void __launch_bounds__(256) k_wp_combine(const int* __restrict__ P, u32 Np, u32 N, u32 t_rows, size_t os, long long* __restrict__ out) {
    const u32 t = blockIdx.y, mt = t / WP_MT, r = t % WP_MT;
    const int* hi = P + ((size_t)mt * 2 * WP_MT + r) * Np;
    const int* lo = hi + (size_t)WP_MT * Np;
    for (u32 j = blockIdx.x * blockDim.x + threadIdx.x; j < N; j += gridDim.x * blockDim.x)
        out[(size_t)t * os + j] = 256ll * hi[j] + lo[j];
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
    const u32 Kp = (u32)((K + WP_KT - 1) / WP_KT * WP_KT), Np = (u32)((N + WP_NT - 1) / WP_NT * WP_NT);
    const u32 tiles = (u32)((t_rows + WP_MT - 1) / WP_MT);
    const bool in_place = !in_out && K % WP_KT == 0 && ((uintptr_t)d_w & 15) == 0;
    const size_t a_bytes = (size_t)tiles * 2 * WP_MT * Kp, p_bytes = (size_t)tiles * 2 * WP_MT * Np * 4, b_bytes = in_place ? 0 : (size_t)N * Kp;
    uint8_t* d_a = nullptr;
    int8_t* d_b = nullptr;
    int *d_p = nullptr, *d_flag = nullptr;
    int rc = dev_alloc(c, (void**)&d_a, a_bytes);
    if (!rc) rc = dev_alloc(c, (void**)&d_p, p_bytes);
    if (!rc) rc = dev_alloc(c, (void**)&d_flag, 4);
    if (!rc && b_bytes) rc = dev_alloc(c, (void**)&d_b, b_bytes);
    // the split over K: enough CTAs for two per SM, each with at least four K stages
    const u32 n_tiles = Np / WP_NT, kt_all = Kp / WP_KT;
    // every CTA does the same work, so what counts is how full the last wave of resident CTAs is: the smallest split that
    // fills the waves best, each split keeping at least two K stages
    const u32 slots = (u32)WP_CTAS_PER_SM * (u32)c->sm_count, base = n_tiles * tiles;
    u32 splits = 1;
    double best = 0.0;
    for (u32 sp = 1; sp <= 32 && sp <= (kt_all / 2 ? kt_all / 2 : 1); sp++) {
        const u64 ctas = (u64)base * sp;
        // each further split adds one pass of integer atomics over the 256 x N plane: charged at 3 % of a product's time
        const double eff = (double)ctas / (double)((ctas + slots - 1) / slots * slots) / (1.0 + 0.03 * (sp - 1));
        if (eff > best + 0.02) { best = eff; splits = sp; }
    }
    int flag = 0;
    if (!rc) {
        Timed t(c, HL_T_WITNESS);
        cudaError_t e = cudaMemsetAsync(d_flag, 0, 4, c->stream);
        if (e == cudaSuccess) e = cudaMemsetAsync(d_out, 0, out_len * 8, c->stream);
        if (e == cudaSuccess && splits > 1) e = cudaMemsetAsync(d_p, 0, p_bytes, c->stream);
        if (e == cudaSuccess && b_bytes) e = cudaMemsetAsync(d_b, 0, b_bytes, c->stream);
        if (e == cudaSuccess) {
            k_wp_pack<<<dim3((Kp + 1023) / 1024, tiles * WP_MT), 256, 0, c->stream>>>((const long long*)d_x, xs, (u32)t_rows, (u32)K, Kp, d_a, d_flag);
            e = cudaGetLastError();
            c->stats.kernel_launches++;
        }
        if (e == cudaSuccess && b_bytes) {
            k_wp_repack<<<dim3(Kp / 64, Np / 64), 256, 0, c->stream>>>(d_w, (u32)K, (u32)N, Kp, in_out, d_b);
            e = cudaGetLastError();
            c->stats.kernel_launches++;
        }
        const size_t smem = (size_t)WP_STAGES * (2 * WP_MT + WP_NT) * WP_LD;
        if (e == cudaSuccess) e = cudaFuncSetAttribute(k_wp_gemm, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) {
            k_wp_gemm<<<dim3(n_tiles, splits, tiles), WP_THREADS, smem, c->stream>>>(d_a, in_place ? d_w : d_b, in_place ? K : (size_t)Kp, (u32)N, Kp, Np, d_p);
            e = cudaGetLastError();
            c->stats.kernel_launches++;
        }
        if (e == cudaSuccess) {
            k_wp_combine<<<dim3((unsigned)((N + 1023) / 1024), (unsigned)t_rows), 256, 0, c->stream>>>(d_p, Np, (u32)N, (u32)t_rows, os, (long long*)d_out);
            e = cudaGetLastError();
            c->stats.kernel_launches++;
        }
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "witness product launch", e);
    }
    if (!rc) rc = d2h(c, &flag, d_flag, 4);
    if (!rc) rc = sync(c, "witness_product");
    else cudaStreamSynchronize(c->stream);
    if (d_a) dev_free(c, d_a, a_bytes);
    if (d_p) dev_free(c, d_p, p_bytes);
    if (d_flag) dev_free(c, d_flag, 4);
    if (d_b) dev_free(c, d_b, b_bytes);
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
