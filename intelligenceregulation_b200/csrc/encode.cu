// Row-encoder kernels: persistent CTAs, one row at a time per CTA (see encode_core.cuh).
#define GL_PLAIN_CANONICAL_FORMS 1  // see gl_field.cuh: this file is tuned around the 64-bit C forms
#include "encode_core.cuh"
#include "kernels.h"

namespace {

struct CtaSync {
    __device__ __forceinline__ void operator()() const { __syncthreads(); }
};

__global__ void k_encode_generic(enc::RowArgs a, u32 logn) {
    extern __shared__ u64 smem[];
    u64* S = smem;
    const u32 n = 1u << logn, tid = threadIdx.x, nt = blockDim.x;
    u64* X = a.scratch + (size_t)blockIdx.x * a.T * n;
    for (u32 row = blockIdx.x; row < a.rows; row += gridDim.x) {
        enc::Generic::load(a, row, logn, S, tid, nt);
        __syncthreads();
        for (u32 ln = logn; ln >= 1; ln--) {
            enc::Generic::dif_stage(a, logn, ln, S, tid, nt);
            __syncthreads();
        }
        enc::Generic::coeffs(a, row, logn, S, X, tid, nt);
        __syncthreads();
        for (u32 s = 0; s < (1u << a.logr); s++) {
            enc::Generic::twist(a, logn, s, X, S, tid, nt);
            __syncthreads();
            for (u32 ln = 1; ln <= logn; ln++) {
                enc::Generic::dit_stage(a, logn, ln, S, tid, nt);
                __syncthreads();
            }
            enc::Generic::store(a, row, logn, s, S, tid, nt);
            __syncthreads();
        }
    }
}

template <int LOGN, int THREADS, int FORM = enc::FORM_PCS, bool NARROW = false>
__global__ void __launch_bounds__(THREADS) k_encode_fast(enc::RowArgs a) {
    using F = enc::Fast<LOGN>;
    extern __shared__ u64 smem[];
    u64* S = smem;
    u64* TW = smem + F::N;
    const u32 tid = threadIdx.x;
    u64* X = a.scratch + (size_t)blockIdx.x * a.T * F::N;
    F::load_twiddles(a, TW, tid, THREADS);
    __syncthreads();
    if (a.split) {
        for (u32 unit = blockIdx.x; unit < (a.rows << a.logr); unit += gridDim.x) {
            const u32 row = unit >> a.logr, s = unit & ((1u << a.logr) - 1u);
            F::template row_coeffs<CtaSync, FORM, NARROW>(a, row, S, TW, X, tid, THREADS, CtaSync());
            __syncthreads();
            F::row_residue(a, row, s, S, TW, X, tid, THREADS, CtaSync());
            __syncthreads();
        }
        return;
    }
    for (u32 row = blockIdx.x; row < a.rows; row += gridDim.x) {
        F::template row_coeffs<CtaSync, FORM, NARROW>(a, row, S, TW, X, tid, THREADS, CtaSync());
        __syncthreads();  // the scratch slot is complete and shared memory is free again
        for (u32 s = 0; s < (1u << a.logr); s++) {
            F::row_residue(a, row, s, S, TW, X, tid, THREADS, CtaSync());
            __syncthreads();
        }
    }
}

// packed rows widened in a pass of their own: the shapes the fast path does not cover (rows below 2^8 or above 2^14 words)
__global__ void __launch_bounds__(256) k_widen_rows(const unsigned char* __restrict__ narrow, const u64* __restrict__ row_off,
                                                    const unsigned char* __restrict__ row_w, u64* __restrict__ out, u32 rows, u32 n) {
    const size_t total = (size_t)rows * n;
    for (size_t x = (size_t)blockIdx.x * blockDim.x + threadIdx.x; x < total; x += (size_t)gridDim.x * blockDim.x) {
        const u32 row = (u32)(x / n), i = (u32)(x - (size_t)row * n);
        out[x] = enc::widen_word(narrow + row_off[row], i, row_w[row]);
    }
}

template <int LOGN>
constexpr int fast_threads() {
    constexpr int g = (1 << LOGN) / 16;
    return g < 32 ? 32 : (g > 1024 ? 1024 : g);
}

template <int LOGN, int FORM = enc::FORM_PCS, bool NARROW = false>
cudaError_t launch_fast(const enc::RowArgs& a, int sm_count, size_t scratch_words, cudaStream_t st, int* grid_out) {
    using F = enc::Fast<LOGN>;
    constexpr int T = fast_threads<LOGN>();
    auto kern = k_encode_fast<LOGN, T, FORM, NARROW>;
    size_t smem = (size_t)(F::N + F::TW_WORDS) * 8;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, T, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) per_sm = 1;
    size_t grid = (size_t)sm_count * per_sm;
    const size_t units = a.split ? (size_t)a.rows << a.logr : (size_t)a.rows;
    if (grid > units) grid = units;
    size_t max_by_scratch = scratch_words / ((size_t)a.T * F::N);
    if (grid > max_by_scratch) grid = max_by_scratch;
    if (grid < 1) return cudaErrorInvalidValue;
    *grid_out = (int)grid;
    kern<<<(unsigned)grid, T, smem, st>>>(a);
    return cudaGetLastError();
}

}  // namespace

namespace hlk {

size_t encode_scratch_words(u32 logn, u32 T, int sm_count, u32 rows) {
    // enough for the largest grid any path launches: 32 CTAs per SM at most, one per row (or, for a handful of rows, one per
    // (row, residue): at most one CTA per SM then)
    size_t ctas = (size_t)sm_count * 32;
    if (ctas > rows && rows >= (u32)sm_count) ctas = rows;
    if (rows < (u32)sm_count) ctas = (size_t)sm_count;
    return ctas * T * ((size_t)1 << logn);
}

cudaError_t encode_rows(const enc::RowArgs& a, u32 logn, bool allow_fast, int sm_count, size_t scratch_words,
                        cudaStream_t st, int* path_out) {
    int grid = 0;
    if (a.narrow) {  // packed rows: the widening first pass exists on the fast path only (the caller widens separately otherwise)
        if (!allow_fast || logn < 8 || logn > 14 || a.loga) return cudaErrorInvalidValue;
        if (path_out) *path_out = 2;
        switch (logn) {
            case 8: return launch_fast<8, enc::FORM_PCS, true>(a, sm_count, scratch_words, st, &grid);
            case 9: return launch_fast<9, enc::FORM_PCS, true>(a, sm_count, scratch_words, st, &grid);
            case 10: return launch_fast<10, enc::FORM_PCS, true>(a, sm_count, scratch_words, st, &grid);
            case 11: return launch_fast<11, enc::FORM_PCS, true>(a, sm_count, scratch_words, st, &grid);
            case 12: return launch_fast<12, enc::FORM_PCS, true>(a, sm_count, scratch_words, st, &grid);
            case 13: return launch_fast<13, enc::FORM_PCS, true>(a, sm_count, scratch_words, st, &grid);
            case 14: return launch_fast<14, enc::FORM_PCS, true>(a, sm_count, scratch_words, st, &grid);
        }
    }
    if (allow_fast && logn >= 8 && logn <= 14) {
        if (path_out) *path_out = 1;
        switch (logn) {
            case 8: return launch_fast<8>(a, sm_count, scratch_words, st, &grid);
            case 9: return launch_fast<9>(a, sm_count, scratch_words, st, &grid);
            case 10: return launch_fast<10>(a, sm_count, scratch_words, st, &grid);
            case 11: return launch_fast<11>(a, sm_count, scratch_words, st, &grid);
            case 12: return launch_fast<12>(a, sm_count, scratch_words, st, &grid);
            case 13: return launch_fast<13>(a, sm_count, scratch_words, st, &grid);
            case 14: return launch_fast<14>(a, sm_count, scratch_words, st, &grid);
        }
    }
    if (logn < 1 || logn > 14) return cudaErrorInvalidValue;
    if (path_out) *path_out = 0;
    const u32 n = 1u << logn;
    int threads = (int)(n / 2 < 32 ? 32 : (n / 2 > 1024 ? 1024 : n / 2));
    size_t smem = (size_t)n * 8;
    cudaError_t e = cudaFuncSetAttribute(k_encode_generic, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(smem < 1024 ? 1024 : smem));
    if (e != cudaSuccess) return e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_encode_generic, threads, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) per_sm = 1;
    size_t g = (size_t)sm_count * per_sm;
    if (g > a.rows) g = a.rows;
    size_t max_by_scratch = scratch_words / ((size_t)a.T * n);
    if (g > max_by_scratch) g = max_by_scratch;
    if (g < 1) return cudaErrorInvalidValue;
    k_encode_generic<<<(unsigned)g, threads, smem, st>>>(a, logn);
    return cudaGetLastError();
}

cudaError_t widen_rows(const unsigned char* narrow, const u64* row_off, const unsigned char* row_w, u64* out, u32 rows, u32 n, int sm_count, cudaStream_t st) {
    const size_t total = (size_t)rows * n;
    size_t blocks = (total + 255) / 256, cap = (size_t)sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    k_widen_rows<<<(unsigned)blocks, 256, 0, st>>>(narrow, row_off, row_w, out, rows, n);
    return cudaGetLastError();
}

// the rows of a masking commitment (messages of 2^8 .. 2^11 words): FORM_COSET or FORM_COEF, always the fast path
cudaError_t encode_rows_form(const enc::RowArgs& a, u32 logn, int form, int sm_count, size_t scratch_words, cudaStream_t st) {
    int grid = 0;
    const bool coef = form == enc::FORM_COEF;
    if (form != enc::FORM_COSET && !coef) return cudaErrorInvalidValue;
    switch (logn) {
        case 8: return coef ? launch_fast<8, enc::FORM_COEF>(a, sm_count, scratch_words, st, &grid) : launch_fast<8, enc::FORM_COSET>(a, sm_count, scratch_words, st, &grid);
        case 9: return coef ? launch_fast<9, enc::FORM_COEF>(a, sm_count, scratch_words, st, &grid) : launch_fast<9, enc::FORM_COSET>(a, sm_count, scratch_words, st, &grid);
        case 10: return coef ? launch_fast<10, enc::FORM_COEF>(a, sm_count, scratch_words, st, &grid) : launch_fast<10, enc::FORM_COSET>(a, sm_count, scratch_words, st, &grid);
        case 11: return coef ? launch_fast<11, enc::FORM_COEF>(a, sm_count, scratch_words, st, &grid) : launch_fast<11, enc::FORM_COSET>(a, sm_count, scratch_words, st, &grid);
    }
    return cudaErrorInvalidValue;
}

}  // namespace hlk
