// The opening's two store operations over a resident commitment (pcs/backend.rs:30-60):
// row combinations rho^T M and column gathers.
#include "gl_field.cuh"
#include "kernels.h"

namespace {

constexpr int FOLD_G = 8;        // rho vectors per pass over the matrix
constexpr int FOLD_ROWS = 64;    // rows of rho staged in shared memory at a time
constexpr int FOLD_THREADS = 128;

// out[g][out_off + j] = sum_i rho_g[i] * src[i * ld + j * ir]   (pcs.rs:342-378)
// One thread per column j, up to FOLD_G combinations at once; the matrix is read once per
// batch of FOLD_G vectors, coalesced along j.  Grid: (column tiles, batches of FOLD_G).
__global__ void __launch_bounds__(FOLD_THREADS) k_fold_rows(const u64* __restrict__ src, u32 rows, u32 ncols, size_t ld, u32 ir,
                                                            const u64* __restrict__ rhos /* k x rows x 2 */, u32 k,
                                                            u64* __restrict__ out, u32 out_ld, u32 out_off) {
    __shared__ u64 rho_s[FOLD_G][FOLD_ROWS][2];
    const u32 j = blockIdx.x * blockDim.x + threadIdx.x;
    const u32 g0 = blockIdx.y * FOLD_G;
    const u32 ng = min((u32)FOLD_G, k - g0);
    fp2 acc[FOLD_G];
#pragma unroll
    for (int g = 0; g < FOLD_G; g++) acc[g] = f2(0, 0);
    for (u32 r0 = 0; r0 < rows; r0 += FOLD_ROWS) {
        const u32 nr = min((u32)FOLD_ROWS, rows - r0);
        __syncthreads();
        for (u32 t = threadIdx.x; t < ng * nr * 2; t += blockDim.x) {
            u32 g = t / (nr * 2), rem = t % (nr * 2);
            rho_s[g][rem >> 1][rem & 1] = rhos[((size_t)(g0 + g) * rows + r0) * 2 + rem];
        }
        __syncthreads();
        if (j < ncols) {
            for (u32 i = 0; i < nr; i++) {
                const u64 v = src[(size_t)(r0 + i) * ld + (size_t)j * ir];
#pragma unroll
                for (int g = 0; g < FOLD_G; g++) {
                    if (g < (int)ng) {
                        acc[g].c0 = gl_add(acc[g].c0, gl_mul(rho_s[g][i][0], v));
                        acc[g].c1 = gl_add(acc[g].c1, gl_mul(rho_s[g][i][1], v));
                    }
                }
            }
        }
    }
    if (j < ncols) {
#pragma unroll
        for (int g = 0; g < FOLD_G; g++)
            if (g < (int)ng) {
                u64* o = out + ((size_t)(g0 + g) * out_ld + out_off + j) * 2;
                o[0] = acc[g].c0;
                o[1] = acc[g].c1;
            }
    }
}

// out[c * rows + i] = enc[i * nn + idx[c]]   (pcs.rs:1055-1067; order of idx, duplicates repeated)
__global__ void k_gather_cols(const u64* __restrict__ enc, u32 rows, size_t nn, const u64* __restrict__ idx, u32 nidx,
                              u64* __restrict__ out) {
    const u32 i = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
    if (i >= rows || c >= nidx) return;
    out[(size_t)c * rows + i] = enc[(size_t)i * nn + idx[c]];
}

}  // namespace

namespace hlk {

cudaError_t fold_rows(const u64* src, u32 rows, u32 ncols, size_t ld, u32 ir, const u64* d_rhos, u32 k, u64* d_out,
                      u32 out_ld, u32 out_off, cudaStream_t st) {
    if (k == 0 || ncols == 0) return cudaSuccess;
    dim3 grid((ncols + FOLD_THREADS - 1) / FOLD_THREADS, (k + FOLD_G - 1) / FOLD_G);
    k_fold_rows<<<grid, FOLD_THREADS, 0, st>>>(src, rows, ncols, ld, ir, d_rhos, k, d_out, out_ld, out_off);
    return cudaGetLastError();
}

cudaError_t gather_columns(const u64* enc, u32 rows, size_t nn, const u64* d_idx, u32 nidx, u64* d_out, cudaStream_t st) {
    if (nidx == 0) return cudaSuccess;
    dim3 grid((rows + 127u) / 128u, nidx);
    k_gather_cols<<<grid, 128, 0, st>>>(enc, rows, nn, d_idx, nidx, d_out);
    return cudaGetLastError();
}

}  // namespace hlk
