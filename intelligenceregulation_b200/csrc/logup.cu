// LogUp helper arithmetic and int8 weight folds.
//
// LogUp (hashline/src/private_block/protocol.rs:993-1011 `inverses`, :1928-1933 `table_helper`;
// accuracy_act.rs:55-117 `histogram`, `denominators`): a lookup of pairs (index, output) in a table is proved
// with helper columns h_i = 1 / (alpha - q_i), q_i = (idx_i + off) + beta * out_i + tag, a multiplicity vector
// and table helpers m_v / (alpha - t_v).  The inversions use Montgomery's trick (field.rs:212-227) on eight
// denominators per thread, one field inversion per thread.  Inverses are unique, so the batching changes no
// word; what is kept is the refusal rule: ANY zero denominator refuses the whole vector.
//
// Weight folds (zkp-core/src/mle.rs:157-319 `fold_rows_i8`, `fold_cols_i8` and their deferred forms): exact
// integer sums of u64 coefficient x int8 value, reduced once per output.  The values are biased by +128 so
// that every product is unsigned; the bias term 128 * sum(w) is taken off in the field at the end.
#include "gl_field.cuh"
#include "kernels.h"

namespace {

__global__ void k_logup_hist(const int* __restrict__ idx, size_t nq, u32 table_len, u64* __restrict__ mult, int* __restrict__ err) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nq) return;
    int v = idx[i];
    if (v < 0 || (u32)v >= table_len) { atomicExch(err, 1); return; }
    atomicAdd(mult + v, 1ull);
}

constexpr int LB = 8;  // denominators per thread

// h[i] = scale_i / (base - idx_i - beta * out_i), scale_i = mult[i] or 1; idx NULL means idx_i = i
__global__ void __launch_bounds__(128) k_logup_helpers(const int* __restrict__ idx, const int* __restrict__ outv, size_t nq, fp2 base, fp2 beta,
                                                       const u64* __restrict__ mult, u64* __restrict__ h, int* __restrict__ err) {
    const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x, i0 = t * LB;
    if (i0 >= nq) return;
    const int cnt = (int)(nq - i0 < LB ? nq - i0 : LB);
    fp2 d[LB], pre[LB];
    fp2 acc = f2(1, 0);
    bool zero = false;
#pragma unroll
    for (int j = 0; j < LB; j++) {
        if (j < cnt) {
            long long a = idx ? (long long)idx[i0 + j] : (long long)(i0 + j);
            fp2 q = f2_mul_base(beta, gl_from_i64(outv[i0 + j]));
            q.c0 = gl_add(q.c0, gl_from_i64(a));
            d[j] = f2_sub(base, q);
            zero |= f2_is_zero(d[j]);
        } else {
            d[j] = f2(1, 0);
        }
        pre[j] = acc;
        acc = f2_mul(acc, d[j]);
    }
    if (zero) { atomicExch(err, 1); return; }  // "zero LogUp denominator; discard attempt"
    fp2 inv = f2_inv(acc);
#pragma unroll
    for (int j = LB - 1; j >= 0; j--) {
        if (j < cnt) {
            fp2 r = f2_mul(inv, pre[j]);
            if (mult) r = f2_mul_base(r, gl_canon(mult[i0 + j]));
            *reinterpret_cast<ulonglong2*>(h + 2 * (i0 + j)) = make_ulonglong2(r.c0, r.c1);
        }
        inv = f2_mul(inv, d[j]);
    }
}

// ---- int8 weight folds -----------------------------------------------------------------------
// sum_i w_i * m_i with w_i a canonical u64 and m_i an int8: bias m by +128 so that it is unsigned, split w into
// 32-bit halves, and the two half-sums  S0 = sum lo(w_i) (m_i + 128),  S1 = sum hi(w_i) (m_i + 128)  are plain
// 64-bit accumulations of 32x8-bit products (below 2^40 each): no carries, no reduction, as long as fewer than
// 2^16 terms go into one accumulator before it is folded into the running field value
//   S0 + 2^32 S1 - 128 (W0 + 2^32 W1),   W0 = sum lo(w_i), W1 = sum hi(w_i).
constexpr u32 I8_BLOCK = 1u << 15;

__device__ __forceinline__ u64 i8_fold(u64 s0, u64 s1, u64 w0, u64 w1) {
    // each argument is below 2^56: canonical; the result is the exact signed sum mod p
    const u64 W32 = 1ull << 32;
    u64 s = gl_add(s0, gl_mul(s1, W32)), w = gl_add(w0, gl_mul(w1, W32));
    return gl_sub(s, gl_mul(w, 128));
}

constexpr int FR_ROWS = 128;
// out[j] = sum_i w[i] * M[i][j]; one thread per 4 neighbouring columns (one 32-bit load per row), rows staged
// FR_ROWS at a time in shared memory as (low, high) halves of both components
__global__ void __launch_bounds__(128) k_fold_rows_i8(const signed char* __restrict__ m, u32 rows, u32 cols, const u64* __restrict__ w,
                                                      u64* __restrict__ out) {
    __shared__ uint4 ws[FR_ROWS];  // (lo c0, hi c0, lo c1, hi c1)
    const u32 j4 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const bool vec = (cols & 3u) == 0;
    u64 run[4][2] = {}, s[4][4] = {}, wsum[4] = {};
    u32 since = 0;
    for (u32 r0 = 0; r0 < rows; r0 += FR_ROWS) {
        const u32 nr = min((u32)FR_ROWS, rows - r0);
        __syncthreads();
        for (u32 t = threadIdx.x; t < nr; t += blockDim.x) {
            const u64 a = w[(size_t)(r0 + t) * 2], b = w[(size_t)(r0 + t) * 2 + 1];
            ws[t] = make_uint4((u32)a, (u32)(a >> 32), (u32)b, (u32)(b >> 32));
        }
        __syncthreads();
        if (j4 < cols) {
            for (u32 i = 0; i < nr; i++) {
                const signed char* p = m + (size_t)(r0 + i) * cols + j4;
                u32 packed;
                if (vec) {
                    packed = *reinterpret_cast<const u32*>(p) ^ 0x80808080u;  // +128 on every byte
                } else {
                    packed = 0;
                    for (u32 c = 0; c < 4 && j4 + c < cols; c++) packed |= (u32)((int)p[c] + 128) << (8 * c);
                }
                const uint4 wv = ws[i];
                wsum[0] += wv.x; wsum[1] += wv.y; wsum[2] += wv.z; wsum[3] += wv.w;
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const u32 v = (packed >> (8 * c)) & 0xFFu;
                    s[c][0] += (u64)wv.x * v; s[c][1] += (u64)wv.y * v;
                    s[c][2] += (u64)wv.z * v; s[c][3] += (u64)wv.w * v;
                }
            }
            since += nr;
            if (since + FR_ROWS > I8_BLOCK || r0 + FR_ROWS >= rows) {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    run[c][0] = gl_add(run[c][0], i8_fold(s[c][0], s[c][1], wsum[0], wsum[1]));
                    run[c][1] = gl_add(run[c][1], i8_fold(s[c][2], s[c][3], wsum[2], wsum[3]));
                    s[c][0] = s[c][1] = s[c][2] = s[c][3] = 0;
                }
                wsum[0] = wsum[1] = wsum[2] = wsum[3] = 0;
                since = 0;
            }
        }
    }
    if (j4 < cols) {
#pragma unroll
        for (int c = 0; c < 4; c++)
            if (j4 + c < cols) {
                out[2 * (size_t)(j4 + c)] = run[c][0];
                out[2 * (size_t)(j4 + c) + 1] = run[c][1];
            }
    }
}

__device__ __forceinline__ u64 shfl_xor64(u64 v, int m) {
    u32 lo = __shfl_xor_sync(0xffffffffu, (u32)v, m), hi = __shfl_xor_sync(0xffffffffu, (u32)(v >> 32), m);
    return ((u64)hi << 32) | lo;
}

// out[i] = sum_j c[j] * M[i][j]; one CTA per FC_ROWS rows, its eight warps interleaved over the columns: a lane loads
// c[j] once (coalesced over the lanes) and multiplies it into the bytes of the FC_ROWS rows at column j; warp tree,
// then a shared-memory sum over the warps
constexpr int FC_ROWS = 4;
constexpr int FC_WARPS = 8;
__global__ void __launch_bounds__(32 * FC_WARPS) k_fold_cols_i8(const signed char* __restrict__ m, u32 rows, u32 cols, const u64* __restrict__ c,
                                                                u64* __restrict__ out) {
    __shared__ u64 part[FC_WARPS][FC_ROWS][2];
    const u32 row0 = blockIdx.x * FC_ROWS, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const u32 nr = min((u32)FC_ROWS, rows - row0);
    u64 s[FC_ROWS][4] = {}, ws[4] = {}, run[FC_ROWS][2] = {};
    u32 since = 0;
#pragma unroll 4
    for (u32 j = threadIdx.x; j < cols; j += 32 * FC_WARPS) {
        const ulonglong2 cw = *reinterpret_cast<const ulonglong2*>(c + 2 * (size_t)j);
        const u32 a0 = (u32)cw.x, a1 = (u32)(cw.x >> 32), b0 = (u32)cw.y, b1 = (u32)(cw.y >> 32);
        ws[0] += a0; ws[1] += a1; ws[2] += b0; ws[3] += b1;
#pragma unroll
        for (int r = 0; r < FC_ROWS; r++) {
            if ((u32)r < nr) {
                const u32 v = (u32)((int)m[(size_t)(row0 + r) * cols + j] + 128);
                s[r][0] += (u64)a0 * v; s[r][1] += (u64)a1 * v; s[r][2] += (u64)b0 * v; s[r][3] += (u64)b1 * v;
            }
        }
        if (++since == I8_BLOCK) {
#pragma unroll
            for (int r = 0; r < FC_ROWS; r++) {
                run[r][0] = gl_add(run[r][0], i8_fold(s[r][0], s[r][1], ws[0], ws[1]));
                run[r][1] = gl_add(run[r][1], i8_fold(s[r][2], s[r][3], ws[2], ws[3]));
                s[r][0] = s[r][1] = s[r][2] = s[r][3] = 0;
            }
            ws[0] = ws[1] = ws[2] = ws[3] = 0;
            since = 0;
        }
    }
#pragma unroll
    for (int r = 0; r < FC_ROWS; r++) {
        u64 x0 = gl_add(run[r][0], i8_fold(s[r][0], s[r][1], ws[0], ws[1]));
        u64 x1 = gl_add(run[r][1], i8_fold(s[r][2], s[r][3], ws[2], ws[3]));
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            x0 = gl_add(x0, shfl_xor64(x0, off));
            x1 = gl_add(x1, shfl_xor64(x1, off));
        }
        if (lane == 0) { part[warp][r][0] = x0; part[warp][r][1] = x1; }
    }
    __syncthreads();
    if (threadIdx.x < FC_ROWS * 2 && threadIdx.x / 2 < nr) {
        u64 x = 0;
#pragma unroll
        for (int w = 0; w < FC_WARPS; w++) x = gl_add(x, part[w][threadIdx.x / 2][threadIdx.x & 1]);
        out[2 * (size_t)(row0 + threadIdx.x / 2) + (threadIdx.x & 1)] = x;
    }
}

// The same sum for rows of whole 16-byte groups (cols a multiple of 16, 16-byte aligned matrix): the matrix is read once with
// 16-byte loads, one row per warp, and the coefficients come from shared memory, a tile of FCV_TILE columns at a time (split
// into their 32-bit halves once per CTA, padded by one entry per 16 so that a quarter-warp's 16-byte reads fall in distinct
// banks).  The bias term 128 * sum_j c[j] is the same for every row: one field sum per CTA instead of four integer
// additions per matrix byte.
constexpr int FCV_WARPS = 8;          // rows per CTA
constexpr int FCV_TILE = 2048;        // columns per shared-memory tile
__global__ void __launch_bounds__(32 * FCV_WARPS) k_fold_cols_i8_vec(const signed char* __restrict__ m, u32 rows, u32 cols, const u64* __restrict__ c,
                                                                     u64* __restrict__ out) {
    __shared__ uint4 cs[FCV_TILE + FCV_TILE / 16];
    __shared__ u64 csum_part[FCV_WARPS][2];
    const u32 lane = threadIdx.x & 31, warp = threadIdx.x >> 5, row = blockIdx.x * FCV_WARPS + warp;
    u64 s[4] = {0, 0, 0, 0}, run0 = 0, run1 = 0, cs0 = 0, cs1 = 0;
    u32 since = 0;
    for (u32 t0 = 0; t0 < cols; t0 += FCV_TILE) {
        const u32 nt = min((u32)FCV_TILE, cols - t0);
        __syncthreads();
        for (u32 j = threadIdx.x; j < nt; j += 32 * FCV_WARPS) {
            const ulonglong2 cw = *reinterpret_cast<const ulonglong2*>(c + 2 * (size_t)(t0 + j));
            cs[j + (j >> 4)] = make_uint4((u32)cw.x, (u32)(cw.x >> 32), (u32)cw.y, (u32)(cw.y >> 32));
            cs0 = gl_add(cs0, cw.x);
            cs1 = gl_add(cs1, cw.y);
        }
        __syncthreads();
        if (row < rows) {
            for (u32 j = lane * 16; j < nt; j += 32 * 16) {
                const uint4 mv = *reinterpret_cast<const uint4*>(m + (size_t)row * cols + t0 + j);
                const u32 words[4] = {mv.x ^ 0x80808080u, mv.y ^ 0x80808080u, mv.z ^ 0x80808080u, mv.w ^ 0x80808080u};  // +128 on every byte
                const uint4* ce = cs + j + (j >> 4);
#pragma unroll
                for (int e = 0; e < 16; e++) {
                    const u32 v = (words[e >> 2] >> (8 * (e & 3))) & 0xFFu;
                    const uint4 cv = ce[e];
                    s[0] += (u64)cv.x * v; s[1] += (u64)cv.y * v; s[2] += (u64)cv.z * v; s[3] += (u64)cv.w * v;
                }
                since += 16;
                if (since + 16 > I8_BLOCK) {  // keep every accumulator below 2^56
                    const u64 W32 = 1ull << 32;
                    run0 = gl_add(run0, gl_add(s[0], gl_mul(s[1], W32)));
                    run1 = gl_add(run1, gl_add(s[2], gl_mul(s[3], W32)));
                    s[0] = s[1] = s[2] = s[3] = 0;
                    since = 0;
                }
            }
        }
    }
    // sum_j c[j] over the CTA (each thread staged a share of every tile)
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        cs0 = gl_add(cs0, shfl_xor64(cs0, off));
        cs1 = gl_add(cs1, shfl_xor64(cs1, off));
    }
    if (lane == 0) { csum_part[warp][0] = cs0; csum_part[warp][1] = cs1; }
    __syncthreads();
    const u64 W32 = 1ull << 32;
    u64 x0 = gl_add(run0, gl_add(s[0], gl_mul(s[1], W32))), x1 = gl_add(run1, gl_add(s[2], gl_mul(s[3], W32)));
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        x0 = gl_add(x0, shfl_xor64(x0, off));
        x1 = gl_add(x1, shfl_xor64(x1, off));
    }
    if (lane == 0 && row < rows) {
        u64 t0 = 0, t1 = 0;
#pragma unroll
        for (int w = 0; w < FCV_WARPS; w++) { t0 = gl_add(t0, csum_part[w][0]); t1 = gl_add(t1, csum_part[w][1]); }
        out[2 * (size_t)row] = gl_sub(x0, gl_mul(t0, 128));
        out[2 * (size_t)row + 1] = gl_sub(x1, gl_mul(t1, 128));
    }
}

// out[j] = sum_i w[i] * M[i][j] for a matrix with many rows (a weight matrix folded over its input dimension, mle.rs:157-200): the
// rows are cut into ranges of FRB_RANGE so that the grid fills the machine, a thread owns eight adjacent columns (8-byte loads, a
// CTA reads 2 KB of every row), the range's weights sit in shared memory as 32-bit halves and are broadcast; range z writes its
// bias-corrected partial sums to part[z][cols] and k_fold_i8_sum adds the ranges.
constexpr int FRB_THREADS = 256, FRB_CPT = 8, FRB_RANGE = 64;
__global__ void __launch_bounds__(FRB_THREADS) k_fold_rows_i8_big(const signed char* __restrict__ m, u32 rows, u32 cols, const u64* __restrict__ w,
                                                                  u32 range /* rows per CTA, at most FRB_RANGE */, u64* __restrict__ part) {
    __shared__ uint4 ws[FRB_RANGE];
    __shared__ u64 wsum[2];
    const u32 row_lo = blockIdx.y * range, nr = min(range, rows - row_lo);
    if (threadIdx.x < nr) {
        const u64 a = w[(size_t)(row_lo + threadIdx.x) * 2], b = w[(size_t)(row_lo + threadIdx.x) * 2 + 1];
        ws[threadIdx.x] = make_uint4((u32)a, (u32)(a >> 32), (u32)b, (u32)(b >> 32));
    }
    if (threadIdx.x < 2) {
        u64 t = 0;
        for (u32 i = 0; i < nr; i++) t = gl_add(t, w[(size_t)(row_lo + i) * 2 + threadIdx.x]);
        wsum[threadIdx.x] = t;
    }
    __syncthreads();
    const u32 col = (blockIdx.x * FRB_THREADS + threadIdx.x) * FRB_CPT;
    if (col >= cols) return;
    u64 s[FRB_CPT][4];
#pragma unroll
    for (int e = 0; e < FRB_CPT; e++) s[e][0] = s[e][1] = s[e][2] = s[e][3] = 0;
    const signed char* p = m + (size_t)row_lo * cols + col;
#pragma unroll 8
    for (u32 i = 0; i < nr; i++) {
        const uint2 mv = *reinterpret_cast<const uint2*>(p + (size_t)i * cols);
        const u32 lo = mv.x ^ 0x80808080u, hi = mv.y ^ 0x80808080u;  // +128 on every byte
        const uint4 wv = ws[i];
#pragma unroll
        for (int e = 0; e < FRB_CPT; e++) {
            const u32 v = ((e < 4 ? lo : hi) >> (8 * (e & 3))) & 0xFFu;
            s[e][0] += (u64)wv.x * v; s[e][1] += (u64)wv.y * v; s[e][2] += (u64)wv.z * v; s[e][3] += (u64)wv.w * v;
        }
    }
    const u64 W32 = 1ull << 32, b0 = gl_mul(wsum[0], 128), b1 = gl_mul(wsum[1], 128);
    u64* o = part + ((size_t)blockIdx.y * cols + col) * 2;
#pragma unroll
    for (int e = 0; e < FRB_CPT; e++) {  // at most 64 terms below 2^40 each: canonical words
        o[2 * e] = gl_sub(gl_add(s[e][0], gl_mul(s[e][1], W32)), b0);
        o[2 * e + 1] = gl_sub(gl_add(s[e][2], gl_mul(s[e][3], W32)), b1);
    }
}

__global__ void __launch_bounds__(256) k_fold_i8_sum(const u64* __restrict__ part, u32 ranges, size_t words, u64* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= words) return;
    u64 s = 0;
    for (u32 z = 0; z < ranges; z++) s = gl_add(s, part[(size_t)z * words + i]);
    out[i] = s;
}

}  // namespace

namespace hlk {

cudaError_t logup_histogram(const int* d_idx, size_t nq, u32 table_len, u64* d_mult, int* d_err, cudaStream_t st) {
    cudaError_t e = cudaMemsetAsync(d_mult, 0, (size_t)table_len * 8, st);
    if (e != cudaSuccess || nq == 0) return e;
    k_logup_hist<<<(unsigned)((nq + 255) / 256), 256, 0, st>>>(d_idx, nq, table_len, d_mult, d_err);
    return cudaGetLastError();
}

cudaError_t logup_helpers(const int* d_idx, const int* d_out, size_t nq, fp2 base, fp2 beta, const u64* d_mult, u64* d_h, int* d_err,
                          cudaStream_t st) {
    if (nq == 0) return cudaSuccess;
    size_t threads = (nq + LB - 1) / LB;
    k_logup_helpers<<<(unsigned)((threads + 127) / 128), 128, 0, st>>>(d_idx, d_out, nq, base, beta, d_mult, d_h, d_err);
    return cudaGetLastError();
}

// rows per CTA of the many-row form: enough ranges for two CTAs per SM, between 8 and FRB_RANGE rows each (0: the single-pass
// kernel serves the shape); scratch = ceil(rows / range) x cols Fp2
u32 fold_rows_i8_range(const signed char* d_m, u32 rows, u32 cols, int sm_count) {
    if (rows < 32 || cols % FRB_CPT != 0 || (reinterpret_cast<uintptr_t>(d_m) & 7) != 0) return 0;
    const u32 tiles = (cols / FRB_CPT + FRB_THREADS - 1) / FRB_THREADS;
    u32 range = (u32)(((u64)rows * tiles + 2u * (u32)sm_count - 1) / (2u * (u32)sm_count));
    if (range < 8) range = 8;
    if (range > (u32)FRB_RANGE) range = FRB_RANGE;
    return range;
}

cudaError_t fold_rows_i8_big(const signed char* d_m, u32 rows, u32 cols, const u64* d_w, u64* d_out, u32 range, u64* d_part, cudaStream_t st) {
    const u32 ranges = (rows + range - 1) / range;
    dim3 grid((cols / FRB_CPT + FRB_THREADS - 1) / FRB_THREADS, ranges);
    k_fold_rows_i8_big<<<grid, FRB_THREADS, 0, st>>>(d_m, rows, cols, d_w, range, d_part);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const size_t words = (size_t)cols * 2;
    k_fold_i8_sum<<<(unsigned)((words + 255) / 256), 256, 0, st>>>(d_part, ranges, words, d_out);
    return cudaGetLastError();
}

cudaError_t fold_rows_i8(const signed char* d_m, u32 rows, u32 cols, const u64* d_w, u64* d_out, cudaStream_t st) {
    u32 threads = (cols + 3) / 4;
    k_fold_rows_i8<<<(threads + 127) / 128, 128, 0, st>>>(d_m, rows, cols, d_w, d_out);
    return cudaGetLastError();
}

cudaError_t fold_cols_i8(const signed char* d_m, u32 rows, u32 cols, const u64* d_c, u64* d_out, cudaStream_t st) {
    if (cols % 16 == 0 && (reinterpret_cast<uintptr_t>(d_m) & 15) == 0 && cols >= 512) {
        k_fold_cols_i8_vec<<<(rows + FCV_WARPS - 1) / FCV_WARPS, 32 * FCV_WARPS, 0, st>>>(d_m, rows, cols, d_c, d_out);
        return cudaGetLastError();
    }
    k_fold_cols_i8<<<(rows + FC_ROWS - 1) / FC_ROWS, 32 * FC_WARPS, 0, st>>>(d_m, rows, cols, d_c, d_out);
    return cudaGetLastError();
}

}  // namespace hlk
