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

// 128-bit accumulate of a 64 x 8 bit unsigned product
__device__ __forceinline__ void mac128(u64& lo, u64& hi, u64 w, u32 v) {
    u64 pl = w * v, ph = __umul64hi(w, (u64)v);
    lo += pl;
    hi += ph + (lo < pl ? 1ull : 0ull);
}
__device__ __forceinline__ void add128(u64& lo, u64& hi, u64 l2, u64 h2) {
    lo += l2;
    hi += h2 + (lo < l2 ? 1ull : 0ull);
}
// (sum - 128 * wsum) mod p from the two 128-bit unsigned sums
__device__ __forceinline__ u64 unbias(u64 lo, u64 hi, u64 wlo, u64 whi) {
    u64 s = gl_reduce128(lo, hi), w = gl_reduce128(wlo, whi);
    return gl_sub(s, gl_mul(w, 128));
}

constexpr int FR_ROWS = 128;
// out[j] = sum_i w[i] * M[i][j]; one thread per 4 neighbouring columns, rows staged 128 at a time
__global__ void __launch_bounds__(128) k_fold_rows_i8(const signed char* __restrict__ m, u32 rows, u32 cols, const u64* __restrict__ w,
                                                      u64* __restrict__ out) {
    __shared__ u64 ws[FR_ROWS][2];
    const u32 j4 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    u64 lo[4][2] = {}, hi[4][2] = {}, wl[2] = {}, wh[2] = {};
    for (u32 r0 = 0; r0 < rows; r0 += FR_ROWS) {
        const u32 nr = min((u32)FR_ROWS, rows - r0);
        __syncthreads();
        for (u32 t = threadIdx.x; t < nr * 2; t += blockDim.x) ws[t >> 1][t & 1] = w[(size_t)(r0 + (t >> 1)) * 2 + (t & 1)];
        __syncthreads();
        if (j4 < cols) {
            for (u32 i = 0; i < nr; i++) {
                const signed char* p = m + (size_t)(r0 + i) * cols + j4;
                const u64 w0 = ws[i][0], w1 = ws[i][1];
                add128(wl[0], wh[0], w0, 0);
                add128(wl[1], wh[1], w1, 0);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    if (j4 + c < cols) {
                        u32 v = (u32)((int)p[c] + 128);
                        mac128(lo[c][0], hi[c][0], w0, v);
                        mac128(lo[c][1], hi[c][1], w1, v);
                    }
                }
            }
        }
    }
    if (j4 < cols) {
#pragma unroll
        for (int c = 0; c < 4; c++)
            if (j4 + c < cols) {
                out[2 * (size_t)(j4 + c)] = unbias(lo[c][0], hi[c][0], wl[0], wh[0]);
                out[2 * (size_t)(j4 + c) + 1] = unbias(lo[c][1], hi[c][1], wl[1], wh[1]);
            }
    }
}

__device__ __forceinline__ u64 shfl_xor64(u64 v, int m) {
    u32 lo = __shfl_xor_sync(0xffffffffu, (u32)v, m), hi = __shfl_xor_sync(0xffffffffu, (u32)(v >> 32), m);
    return ((u64)hi << 32) | lo;
}

// out[i] = sum_j c[j] * M[i][j]; one warp per row, lanes stride over the columns, warp tree on the 128-bit sums
__global__ void __launch_bounds__(256) k_fold_cols_i8(const signed char* __restrict__ m, u32 rows, u32 cols, const u64* __restrict__ c,
                                                      u64* __restrict__ out) {
    const u32 row = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const signed char* p = m + (size_t)row * cols;
    u64 lo[2] = {}, hi[2] = {}, wl[2] = {}, wh[2] = {};
    for (u32 j = lane; j < cols; j += 32) {
        const ulonglong2 cw = *reinterpret_cast<const ulonglong2*>(c + 2 * (size_t)j);
        u32 v = (u32)((int)p[j] + 128);
        mac128(lo[0], hi[0], cw.x, v);
        mac128(lo[1], hi[1], cw.y, v);
        add128(wl[0], wh[0], cw.x, 0);
        add128(wl[1], wh[1], cw.y, 0);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
        for (int k = 0; k < 2; k++) {
            add128(lo[k], hi[k], shfl_xor64(lo[k], off), shfl_xor64(hi[k], off));
            add128(wl[k], wh[k], shfl_xor64(wl[k], off), shfl_xor64(wh[k], off));
        }
    }
    if (lane == 0) {
        out[2 * (size_t)row] = unbias(lo[0], hi[0], wl[0], wh[0]);
        out[2 * (size_t)row + 1] = unbias(lo[1], hi[1], wl[1], wh[1]);
    }
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

cudaError_t fold_rows_i8(const signed char* d_m, u32 rows, u32 cols, const u64* d_w, u64* d_out, cudaStream_t st) {
    u32 threads = (cols + 3) / 4;
    k_fold_rows_i8<<<(threads + 127) / 128, 128, 0, st>>>(d_m, rows, cols, d_w, d_out);
    return cudaGetLastError();
}

cudaError_t fold_cols_i8(const signed char* d_m, u32 rows, u32 cols, const u64* d_c, u64* d_out, cudaStream_t st) {
    k_fold_cols_i8<<<(rows + 7) / 8, 256, 0, st>>>(d_m, rows, cols, d_c, d_out);
    return cudaGetLastError();
}

}  // namespace hlk
