// The opening's two store operations over a resident commitment (pcs/backend.rs:30-60):
// row combinations rho^T M and column gathers.
#include "gl_field.cuh"
#include "kernels.h"

namespace {

// ---------------------------------------------------------------------------------------------
// out[g][out_off + j] = sum_i rho_g[i] * src[i * ld + j * ir]   (pcs.rs:342-378, 976-1000)
//
// A dense (2k x rows) by (rows x ncols) product over the field: 3.2 G multiply-adds for the 8B block's
// opening (38 vectors, 2,504 rows, 16,664 columns).  Reducing every product would cost ~27 instructions
// each, so products are accumulated as plain integers and reduced once per block of rows:
// a matrix word is cut into limbs of 22 + 22 + 20 bits, a rho component into two 32-bit halves, and the
// six limb products (each < 2^54) are summed in six 64-bit accumulators with 32x32+64 multiply-adds and
// no carry handling at all.  After FOLD_BLOCK = 256 rows (sums < 2^62) the six accumulators are folded
// into the running field value with their weights 2^(22a + 32b).  Field addition is exact, so the words
// are those of the reference's per-element loop (its zero skips only save work).
//
// One thread owns one column and FOLD_RPT rho vectors (2 x FOLD_RPT base-field components); a CTA is
// 128 columns x FOLD_GROUPS groups of vectors, so that the groups' reads of the same matrix words are
// served by L1.  Grid: (column tiles, batches of FOLD_RPT * FOLD_GROUPS vectors).
// ---------------------------------------------------------------------------------------------
constexpr int FOLD_COLS = 128;
constexpr int FOLD_GROUPS = 4;
constexpr int FOLD_RPT = 2;                           // rho vectors per thread
constexpr int FOLD_G = FOLD_RPT * FOLD_GROUPS;        // rho vectors per CTA
constexpr int FOLD_BLOCK = 256;                       // rows between reductions
constexpr int FOLD_THREADS = FOLD_COLS * FOLD_GROUPS;

// Two column segments in one launch (the message columns and the pad columns of a hiding opening), so that
// the narrow pad segment's few CTAs run beside the wide segment's instead of as a tail of their own.
struct FoldSeg {
    const u64* src;
    size_t ld;
    u32 ncols, ir, out_off, tiles;
};

// With gridDim.z > 1 the rows are cut into gridDim.z ranges (a few dense vectors alone leave most of the machine without
// loads in flight): range z writes its partial combination to out + z * k * out_ld (vector order, no map) and
// k_fold_sum adds the ranges.
__global__ void __launch_bounds__(FOLD_THREADS) k_fold_rows(FoldSeg seg0, FoldSeg seg1, u32 rows,
                                                            const u64* __restrict__ rhos /* k x rows x 2 */, u32 k,
                                                            const u32* __restrict__ out_map /* vector -> output row, or NULL */,
                                                            u64* __restrict__ out, u32 out_ld) {
    __shared__ uint2 rho_s[FOLD_BLOCK][FOLD_G * 2];  // [row][vector * 2 + component] = (low half, high half)
    const bool second = blockIdx.x >= seg0.tiles;
    const u64* __restrict__ src = second ? seg1.src : seg0.src;
    const size_t ld = second ? seg1.ld : seg0.ld;
    const u32 ncols = second ? seg1.ncols : seg0.ncols, ir = second ? seg1.ir : seg0.ir, out_off = second ? seg1.out_off : seg0.out_off;
    const u32 tile = second ? blockIdx.x - seg0.tiles : blockIdx.x;
    const u32 col = tile * FOLD_COLS + (threadIdx.x % FOLD_COLS), grp = threadIdx.x / FOLD_COLS;
    const u32 g0 = blockIdx.y * FOLD_G;
    const u32 ng = min((u32)FOLD_G, k - g0);
    constexpr int NC = FOLD_RPT * 2;  // components per thread
    u64 run[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) run[c] = 0;
    // weights of the six limb products: 2^(22 a + 32 b), a = 0..2, b = 0..1
    const u64 W22 = 1ull << 22, W44 = 1ull << 44, W32 = 1ull << 32, W54 = 1ull << 54;
    const u64 W76 = gl_reduce128(0, 1ull << 12);  // 2^76 mod p
    const u32 per_z = (rows + gridDim.z - 1) / gridDim.z;
    const u32 row_lo = blockIdx.z * per_z, row_hi = min(rows, row_lo + per_z);
    for (u32 r0 = row_lo; r0 < row_hi; r0 += FOLD_BLOCK) {
        const u32 nr = min((u32)FOLD_BLOCK, row_hi - r0);
        __syncthreads();
        for (u32 t = threadIdx.x; t < nr * FOLD_G * 2; t += FOLD_THREADS) {
            const u32 i = t / (FOLD_G * 2), gc = t % (FOLD_G * 2), g = gc >> 1;
            u64 w = g < ng ? rhos[((size_t)(g0 + g) * rows + r0 + i) * 2 + (gc & 1)] : 0ull;
            rho_s[i][gc] = make_uint2((u32)w, (u32)(w >> 32));
        }
        __syncthreads();
        if (col < ncols && grp * FOLD_RPT < ng) {
            u64 acc[NC][6];
#pragma unroll
            for (int c = 0; c < NC; c++)
#pragma unroll
                for (int x = 0; x < 6; x++) acc[c][x] = 0;
            const u64* p = src + (size_t)r0 * ld + (size_t)col * ir;
            constexpr int PF = 8;  // rows fetched ahead: eight independent loads in flight per thread
            u64 nxt[PF];
#pragma unroll
            for (int x = 0; x < PF; x++) nxt[x] = (u32)x < nr ? p[(size_t)x * ld] : 0ull;
            for (u32 i0 = 0; i0 < nr; i0 += PF) {
                u64 cur[PF];
#pragma unroll
                for (int x = 0; x < PF; x++) cur[x] = nxt[x];
#pragma unroll
                for (int x = 0; x < PF; x++) nxt[x] = i0 + PF + x < nr ? p[(size_t)(i0 + PF + x) * ld] : 0ull;
#pragma unroll
                for (int x = 0; x < PF; x++) {
                    if (i0 + x < nr) {
                        const u64 v = cur[x];
                        const u32 v0 = (u32)v & 0x3FFFFFu, v1 = (u32)(v >> 22) & 0x3FFFFFu, v2 = (u32)(v >> 44);
                        // an opening's group weights are zero outside their claims' rows (pcs.rs:851-891): skip those
                        // rows for this thread's vectors; the test is uniform over the warp
                        u32 any = 0;
#pragma unroll
                        for (int c = 0; c < NC; c++) any |= rho_s[i0 + x][grp * NC + c].x | rho_s[i0 + x][grp * NC + c].y;
                        if (any == 0) continue;
#pragma unroll
                        for (int c = 0; c < NC; c++) {
                            const uint2 r = rho_s[i0 + x][grp * NC + c];
                            acc[c][0] += (u64)v0 * r.x;
                            acc[c][1] += (u64)v1 * r.x;
                            acc[c][2] += (u64)v2 * r.x;
                            acc[c][3] += (u64)v0 * r.y;
                            acc[c][4] += (u64)v1 * r.y;
                            acc[c][5] += (u64)v2 * r.y;
                        }
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < NC; c++) {  // every accumulator is below 2^62 < p: already a canonical word
                u64 s = acc[c][0];
                s = gl_add(s, gl_mul(acc[c][1], W22));
                s = gl_add(s, gl_mul(acc[c][2], W44));
                s = gl_add(s, gl_mul(acc[c][3], W32));
                s = gl_add(s, gl_mul(acc[c][4], W54));
                s = gl_add(s, gl_mul(acc[c][5], W76));
                run[c] = gl_add(run[c], s);
            }
        }
    }
    if (col < ncols) {
#pragma unroll
        for (int v = 0; v < FOLD_RPT; v++) {
            const u32 g = grp * FOLD_RPT + v;
            if (g < ng) {
                const size_t orow = gridDim.z > 1 ? (size_t)blockIdx.z * k + g0 + g : (size_t)(out_map ? out_map[g0 + g] : g0 + g);
                u64* o = out + (orow * out_ld + out_off + col) * 2;
                o[0] = run[2 * v];
                o[1] = run[2 * v + 1];
            }
        }
    }
}

// One or two dense vectors alone (an opening's proximity vector beside its sparse group vectors): the work is one pass over
// the matrix, so the kernel is laid out for the memory system instead of for reuse: a thread owns two adjacent columns
// (16-byte loads), a CTA 512 contiguous columns of a row (4 KB), the rows are cut into gridDim.y short ranges so that every
// SM has several CTAs' loads in flight, eight rows fetched ahead per thread.  Same limb arithmetic as k_fold_rows; a range is
// at most FOLD_BLOCK rows, so the integer sums are folded once.  Contiguous sources only (ir = 1).
constexpr int FEW_THREADS = 256;
constexpr int FEW_COLS = 2 * FEW_THREADS;
template <int KV>
__global__ void __launch_bounds__(FEW_THREADS) k_fold_rows_few(FoldSeg seg0, FoldSeg seg1, u32 rows, u32 per_z, const u64* __restrict__ rhos, u32 k,
                                                               u64* __restrict__ part, u32 out_ld) {
    __shared__ uint2 rho_s[FOLD_BLOCK][KV * 2];
    const bool second = blockIdx.x >= seg0.tiles;
    const u64* __restrict__ src = second ? seg1.src : seg0.src;
    const size_t ld = second ? seg1.ld : seg0.ld;
    const u32 ncols = second ? seg1.ncols : seg0.ncols, out_off = second ? seg1.out_off : seg0.out_off;
    const u32 tile = second ? blockIdx.x - seg0.tiles : blockIdx.x;
    const u32 col = tile * FEW_COLS + 2 * threadIdx.x;
    const u32 row_lo = blockIdx.y * per_z, row_hi = min(rows, row_lo + per_z), nr = row_hi > row_lo ? row_hi - row_lo : 0;
    for (u32 t = threadIdx.x; t < nr * KV * 2; t += FEW_THREADS) {
        const u32 i = t / (KV * 2), gc = t % (KV * 2);
        const u64 w = rhos[((size_t)(gc >> 1) * rows + row_lo + i) * 2 + (gc & 1)];
        rho_s[i][gc] = make_uint2((u32)w, (u32)(w >> 32));
    }
    __syncthreads();
    constexpr int NC = KV * 2;
    u64 acc[2][NC][6];
#pragma unroll
    for (int e = 0; e < 2; e++)
#pragma unroll
        for (int c = 0; c < NC; c++)
#pragma unroll
            for (int x = 0; x < 6; x++) acc[e][c][x] = 0;
    if (col < ncols) {
        const bool two = col + 1 < ncols;  // ncols and ld are even for every store; the odd tail is kept correct anyway
        const u64* p = src + (size_t)row_lo * ld + col;
        constexpr int PF = 8;
        ulonglong2 nxt[PF];
        auto fetch = [&](u32 r) -> ulonglong2 {
            if (r >= nr) return make_ulonglong2(0, 0);
            const u64* q = p + (size_t)r * ld;
            if (two && ((reinterpret_cast<uintptr_t>(q) & 15) == 0)) return *reinterpret_cast<const ulonglong2*>(q);
            return make_ulonglong2(q[0], two ? q[1] : 0ull);
        };
#pragma unroll
        for (int x = 0; x < PF; x++) nxt[x] = fetch((u32)x);
        for (u32 i0 = 0; i0 < nr; i0 += PF) {
            ulonglong2 cur[PF];
#pragma unroll
            for (int x = 0; x < PF; x++) cur[x] = nxt[x];
#pragma unroll
            for (int x = 0; x < PF; x++) nxt[x] = fetch(i0 + PF + x);
#pragma unroll
            for (int x = 0; x < PF; x++) {
                if (i0 + x < nr) {
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const u64 v = e ? cur[x].y : cur[x].x;
                        const u32 v0 = (u32)v & 0x3FFFFFu, v1 = (u32)(v >> 22) & 0x3FFFFFu, v2 = (u32)(v >> 44);
#pragma unroll
                        for (int c = 0; c < NC; c++) {
                            const uint2 r = rho_s[i0 + x][c];
                            acc[e][c][0] += (u64)v0 * r.x;
                            acc[e][c][1] += (u64)v1 * r.x;
                            acc[e][c][2] += (u64)v2 * r.x;
                            acc[e][c][3] += (u64)v0 * r.y;
                            acc[e][c][4] += (u64)v1 * r.y;
                            acc[e][c][5] += (u64)v2 * r.y;
                        }
                    }
                }
            }
        }
        const u64 W22 = 1ull << 22, W44 = 1ull << 44, W32 = 1ull << 32, W54 = 1ull << 54;
        const u64 W76 = gl_reduce128(0, 1ull << 12);  // 2^76 mod p
#pragma unroll
        for (int e = 0; e < 2; e++) {
            if (col + e < ncols) {
#pragma unroll
                for (int g = 0; g < KV; g++) {
                    if ((u32)g < k) {
                        u64* o = part + ((((size_t)blockIdx.y * k + g) * out_ld) + out_off + col + e) * 2;
#pragma unroll
                        for (int cc = 0; cc < 2; cc++) {
                            const u64* a = acc[e][2 * g + cc];
                            u64 sum = a[0];
                            sum = gl_add(sum, gl_mul(a[1], W22));
                            sum = gl_add(sum, gl_mul(a[2], W44));
                            sum = gl_add(sum, gl_mul(a[3], W32));
                            sum = gl_add(sum, gl_mul(a[4], W54));
                            sum = gl_add(sum, gl_mul(a[5], W76));
                            o[cc] = sum;
                        }
                    }
                }
            }
        }
    }
}

// out[map[g]][j] = sum_z part[z][g][j]
__global__ void __launch_bounds__(256) k_fold_sum(const u64* __restrict__ part, u32 splits, u32 k, u32 out_ld, const u32* __restrict__ out_map,
                                                  u64* __restrict__ out) {
    const size_t words = (size_t)out_ld * 2, i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const u32 g = blockIdx.y;
    if (i >= words) return;
    u64 s = 0;
    for (u32 z = 0; z < splits; z++) s = gl_add(s, part[((size_t)z * k + g) * words + i]);
    out[(size_t)(out_map ? out_map[g] : g) * words + i] = s;
}

// The same combination for a vector that is zero outside a few rows (an opening's group weights live on their claims'
// rows only, pcs.rs:851-891): the rows and weights arrive as a list, one thread per column walks it.  Products are
// summed as 128-bit integers with a wrap count and reduced once per component (2^128 = -2^32 mod p).
constexpr int SPARSE_COLS = 256;
__global__ void __launch_bounds__(SPARSE_COLS) k_fold_sparse(FoldSeg seg0, FoldSeg seg1, const u32* __restrict__ off /* vectors + 1 */,
                                                            const u32* __restrict__ srow, const u64* __restrict__ sw /* 2 per entry */,
                                                            const u32* __restrict__ out_map, u64* __restrict__ out, u32 out_ld) {
    const bool second = blockIdx.x >= seg0.tiles;
    const FoldSeg& sg = second ? seg1 : seg0;
    const u32 col = (second ? blockIdx.x - seg0.tiles : blockIdx.x) * SPARSE_COLS + threadIdx.x;
    if (col >= sg.ncols) return;
    const u32 v = blockIdx.y;
    const u64* p = sg.src + (size_t)col * sg.ir;
    u64 lo0 = 0, hi0 = 0, w0 = 0, lo1 = 0, hi1 = 0, w1 = 0;
    for (u32 e = off[v]; e < off[v + 1]; e++) {
        const u64 d = p[(size_t)srow[e] * sg.ld];
        const gl_wide p0 = gl_mulw(sw[2 * (size_t)e], d), p1 = gl_mulw(sw[2 * (size_t)e + 1], d);
        u64 t = lo0 + p0.lo, c = t < lo0; lo0 = t;
        t = hi0 + p0.hi; u64 c2 = t < hi0; hi0 = t + c; c2 += hi0 < t; w0 += c2;
        t = lo1 + p1.lo; c = t < lo1; lo1 = t;
        t = hi1 + p1.hi; c2 = t < hi1; hi1 = t + c; c2 += hi1 < t; w1 += c2;
    }
    const u64 two128 = 0xFFFFFFFE00000001ull;  // 2^128 mod p
    u64* o = out + ((size_t)out_map[v] * out_ld + sg.out_off + col) * 2;
    o[0] = gl_add(gl_reduce128(lo0, hi0), gl_mul(w0, two128));
    o[1] = gl_add(gl_reduce128(lo1, hi1), gl_mul(w1, two128));
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

// the one-pass form for one or two dense vectors over contiguous rows: its number of row ranges (0 = not applicable)
u32 fold_few_ranges(u32 rows, u32 ncols, u32 ncols2, u32 k, u32 ir, int sm_count) {
    if (k == 0 || k > 2 || ir != 1 || rows < 64) return 0;
    const u32 tiles = (ncols + FEW_COLS - 1) / FEW_COLS + (ncols2 + FEW_COLS - 1) / FEW_COLS;
    u32 z = (8u * (u32)sm_count + tiles - 1) / tiles;           // about eight CTAs per SM
    const u32 least = (rows + FOLD_BLOCK - 1) / FOLD_BLOCK;     // a range is at most FOLD_BLOCK rows
    if (z < least) z = least;
    if (z > rows / 16) z = rows / 16 ? rows / 16 : 1;
    if ((rows + z - 1) / z > (u32)FOLD_BLOCK) return 0;
    return z;
}

cudaError_t fold_rows_few(const u64* src, u32 rows, u32 ncols, size_t ld, const u64* src2, u32 ncols2, size_t ld2, const u64* d_rhos, u32 k,
                          const u32* d_out_map, u64* d_out, u32 out_ld, u32 ranges, u64* d_part, cudaStream_t st) {
    FoldSeg a{src, ld, ncols, 1u, 0u, (ncols + FEW_COLS - 1) / FEW_COLS};
    FoldSeg b{src2, ld2, src2 ? ncols2 : 0u, 1u, ncols, src2 ? (ncols2 + FEW_COLS - 1) / FEW_COLS : 0u};
    const u32 per_z = (rows + ranges - 1) / ranges;
    dim3 grid(a.tiles + b.tiles, ranges);
    if (k == 1) k_fold_rows_few<1><<<grid, FEW_THREADS, 0, st>>>(a, b, rows, per_z, d_rhos, k, d_part, out_ld);
    else k_fold_rows_few<2><<<grid, FEW_THREADS, 0, st>>>(a, b, rows, per_z, d_rhos, k, d_part, out_ld);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    k_fold_sum<<<dim3((out_ld * 2 + 255) / 256, k), 256, 0, st>>>(d_part, ranges, k, out_ld, d_out_map, d_out);
    return cudaGetLastError();
}

u32 fold_row_splits(u32 rows, u32 ncols, u32 ncols2, u32 k, int sm_count) {
    const u32 ctas = ((ncols + FOLD_COLS - 1) / FOLD_COLS + (ncols2 + FOLD_COLS - 1) / FOLD_COLS) * ((k + FOLD_G - 1) / FOLD_G);
    if (ctas == 0 || rows < 512) return 1;
    u32 s = (8u * (u32)sm_count + ctas - 1) / ctas;  // eight CTAs' worth of loads in flight per SM
    if (s > 16) s = 16;
    if (s > rows / 128) s = rows / 128;
    return s < 2 ? 1 : s;
}

cudaError_t fold_rows(const u64* src, u32 rows, u32 ncols, size_t ld, u32 ir, const u64* src2, u32 ncols2, size_t ld2,
                      const u64* d_rhos, u32 k, const u32* d_out_map, u64* d_out, u32 out_ld, cudaStream_t st, u32 splits, u64* d_part) {
    if (k == 0 || ncols == 0) return cudaSuccess;
    FoldSeg a{src, ld, ncols, ir, 0u, (ncols + FOLD_COLS - 1) / FOLD_COLS};
    FoldSeg b{src2, ld2, src2 ? ncols2 : 0u, 1u, ncols, src2 ? (ncols2 + FOLD_COLS - 1) / FOLD_COLS : 0u};
    if (splits < 2 || !d_part) {
        dim3 grid(a.tiles + b.tiles, (k + FOLD_G - 1) / FOLD_G);
        k_fold_rows<<<grid, FOLD_THREADS, 0, st>>>(a, b, rows, d_rhos, k, d_out_map, d_out, out_ld);
        return cudaGetLastError();
    }
    dim3 grid(a.tiles + b.tiles, (k + FOLD_G - 1) / FOLD_G, splits);
    k_fold_rows<<<grid, FOLD_THREADS, 0, st>>>(a, b, rows, d_rhos, k, nullptr, d_part, out_ld);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    k_fold_sum<<<dim3((out_ld * 2 + 255) / 256, k), 256, 0, st>>>(d_part, splits, k, out_ld, d_out_map, d_out);
    return cudaGetLastError();
}

cudaError_t fold_rows_sparse(const u64* src, u32 ncols, size_t ld, u32 ir, const u64* src2, u32 ncols2, size_t ld2, const u32* d_off,
                             const u32* d_rows, const u64* d_weights, u32 k, const u32* d_out_map, u64* d_out, u32 out_ld, cudaStream_t st) {
    if (k == 0 || ncols == 0) return cudaSuccess;
    FoldSeg a{src, ld, ncols, ir, 0u, (ncols + SPARSE_COLS - 1) / SPARSE_COLS};
    FoldSeg b{src2, ld2, src2 ? ncols2 : 0u, 1u, ncols, src2 ? (ncols2 + SPARSE_COLS - 1) / SPARSE_COLS : 0u};
    dim3 grid(a.tiles + b.tiles, k);
    k_fold_sparse<<<grid, SPARSE_COLS, 0, st>>>(a, b, d_off, d_rows, d_weights, d_out_map, d_out, out_ld);
    return cudaGetLastError();
}

cudaError_t gather_columns(const u64* enc, u32 rows, size_t nn, const u64* d_idx, u32 nidx, u64* d_out, cudaStream_t st) {
    if (nidx == 0) return cudaSuccess;
    dim3 grid((rows + 127u) / 128u, nidx);
    k_gather_cols<<<grid, 128, 0, st>>>(enc, rows, nn, d_idx, nidx, d_out);
    return cudaGetLastError();
}

}  // namespace hlk
