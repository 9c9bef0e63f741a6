// C ABI: LogUp helper columns / multiplicities and the int8 weight folds.
#include "api_internal.h"

using namespace hlapi;

namespace hlk {
cudaError_t logup_histogram(const int* d_idx, size_t nq, u32 table_len, u64* d_mult, int* d_err, cudaStream_t st);
cudaError_t logup_helpers(const int* d_idx, const int* d_out, size_t nq, fp2 base, fp2 beta, const u64* d_mult, u64* d_h, int* d_err,
                          cudaStream_t st);
cudaError_t fold_rows_i8(const signed char* d_m, u32 rows, u32 cols, const u64* d_w, u64* d_out, cudaStream_t st);
u32 fold_rows_i8_range(const signed char* d_m, u32 rows, u32 cols, int sm_count);
cudaError_t fold_rows_i8_big(const signed char* d_m, u32 rows, u32 cols, const u64* d_w, u64* d_out, u32 range, u64* d_part, cudaStream_t st);
cudaError_t fold_cols_i8(const signed char* d_m, u32 rows, u32 cols, const u64* d_c, u64* d_out, cudaStream_t st);
}  // namespace hlk

extern "C" {

int hl_b200_logup_histogram(hl_ctx* c, const int32_t* idx, size_t nq, size_t table_len, uint64_t* mult) {
    if (!c || !mult || (nq && !idx) || table_len == 0 || table_len > (1u << 30)) return fail(c, HL_B200_ERR_ARG, "logup_histogram: argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    int *d_idx = nullptr, *d_err = nullptr, h_err = 0;
    u64* d_mult = nullptr;
    int rc = dev_alloc(c, (void**)&d_idx, nq * 4);
    if (!rc) rc = dev_alloc(c, (void**)&d_mult, table_len * 8);
    if (!rc) rc = dev_alloc(c, (void**)&d_err, 4);
    if (!rc) rc = h2d(c, d_idx, idx, nq * 4);
    if (!rc && cudaMemsetAsync(d_err, 0, 4, c->stream) != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "flag clear");
    if (!rc) {
        Timed t(c, HL_T_LOGUP);
        cudaError_t e = hlk::logup_histogram(d_idx, nq, (u32)table_len, d_mult, d_err, c->stream);
        c->stats.kernel_launches++;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "histogram launch", e);
    }
    if (!rc) rc = d2h(c, mult, d_mult, table_len * 8);
    if (!rc) rc = d2h(c, &h_err, d_err, 4);
    if (!rc) rc = sync(c, "logup_histogram");
    dev_free(c, d_idx, nq * 4); dev_free(c, d_mult, table_len * 8); dev_free(c, d_err, 4);
    if (!rc && h_err) rc = fail(c, HL_B200_ERR_ARG, "logup_histogram: a query index lies outside the table");
    return rc;
}

int hl_b200_logup_helpers(hl_ctx* c, const int32_t* idx, const int32_t* outv, size_t n, const uint64_t alpha[2],
                          const uint64_t beta[2], const uint64_t tag[2], int64_t idx_off, const uint64_t* mult, uint64_t* h) {
    if (!c || !outv || !alpha || !beta || !tag || !h) return fail(c, HL_B200_ERR_ARG, "logup_helpers: null argument");
    if (n == 0) return HL_B200_OK;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    // alpha - (idx + off + beta out + tag) = (alpha - tag - off) - idx - beta out, every term formed in the field
    fp2 base = f2_sub(f2(alpha[0], alpha[1]), f2(tag[0], tag[1]));
    base.c0 = gl_sub(base.c0, gl_from_i64(idx_off));
    int *d_idx = nullptr, *d_out = nullptr, *d_err = nullptr, h_err = 0;
    u64 *d_mult = nullptr, *d_h = nullptr;
    int rc = dev_alloc(c, (void**)&d_out, n * 4);
    if (!rc && idx) rc = dev_alloc(c, (void**)&d_idx, n * 4);
    if (!rc && mult) rc = dev_alloc(c, (void**)&d_mult, n * 8);
    if (!rc) rc = dev_alloc(c, (void**)&d_h, n * 16);
    if (!rc) rc = dev_alloc(c, (void**)&d_err, 4);
    if (!rc) rc = h2d(c, d_out, outv, n * 4);
    if (!rc && idx) rc = h2d(c, d_idx, idx, n * 4);
    if (!rc && mult) rc = h2d(c, d_mult, mult, n * 8);
    if (!rc && cudaMemsetAsync(d_err, 0, 4, c->stream) != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "flag clear");
    if (!rc) {
        Timed t(c, HL_T_LOGUP);
        cudaError_t e = hlk::logup_helpers(d_idx, d_out, n, base, f2(beta[0], beta[1]), d_mult, d_h, d_err, c->stream);
        c->stats.kernel_launches++;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "helper launch", e);
    }
    if (!rc) rc = d2h(c, &h_err, d_err, 4);
    if (!rc) rc = sync(c, "logup_helpers");
    if (!rc && h_err) rc = fail(c, HL_B200_ERR_ZERO, "zero LogUp denominator; discard attempt");
    if (!rc) rc = d2h(c, h, d_h, n * 16);
    if (!rc) rc = sync(c, "logup_helpers");
    dev_free(c, d_out, n * 4);
    if (d_idx) dev_free(c, d_idx, n * 4);
    if (d_mult) dev_free(c, d_mult, n * 8);
    dev_free(c, d_h, n * 16); dev_free(c, d_err, 4);
    return rc;
}

static int fold_i8(hl_ctx* c, bool by_rows, const int8_t* m, size_t rows, size_t cols, const uint64_t* w, uint64_t* out) {
    if (!c || !m || !w || !out || rows == 0 || cols == 0 || rows > 0x7FFFFFFFu || cols > 0x7FFFFFFFu) return fail(c, HL_B200_ERR_ARG, "fold_i8: argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    const size_t nw = by_rows ? rows : cols, no = by_rows ? cols : rows;
    signed char* d_m = nullptr;
    u64 *d_w = nullptr, *d_o = nullptr;
    int rc = dev_alloc(c, (void**)&d_m, rows * cols);
    if (!rc) rc = dev_alloc(c, (void**)&d_w, nw * 16);
    if (!rc) rc = dev_alloc(c, (void**)&d_o, no * 16);
    if (!rc) rc = h2d(c, d_m, m, rows * cols);
    if (!rc) rc = h2d(c, d_w, w, nw * 16);
    const u32 range = !rc && by_rows ? hlk::fold_rows_i8_range(d_m, (u32)rows, (u32)cols, c->sm_count) : 0;
    const u32 ranges = range ? (u32)((rows + range - 1) / range) : 0;
    u64* d_part = nullptr;
    if (!rc && ranges) rc = dev_alloc(c, (void**)&d_part, (size_t)ranges * cols * 16);
    if (!rc) {
        Timed t(c, HL_T_FOLD);
        cudaError_t e = ranges    ? hlk::fold_rows_i8_big(d_m, (u32)rows, (u32)cols, d_w, d_o, range, d_part, c->stream)
                        : by_rows ? hlk::fold_rows_i8(d_m, (u32)rows, (u32)cols, d_w, d_o, c->stream)
                                  : hlk::fold_cols_i8(d_m, (u32)rows, (u32)cols, d_w, d_o, c->stream);
        c->stats.kernel_launches += ranges ? 2 : 1;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "int8 fold launch", e);
    }
    if (!rc) rc = d2h(c, out, d_o, no * 16);
    if (!rc) rc = sync(c, "fold_i8");
    if (d_part) dev_free(c, d_part, (size_t)ranges * cols * 16);
    dev_free(c, d_m, rows * cols); dev_free(c, d_w, nw * 16); dev_free(c, d_o, no * 16);
    return rc;
}

int hl_b200_fold_rows_i8(hl_ctx* c, const int8_t* m, size_t rows, size_t cols, const uint64_t* w, uint64_t* out) {
    return fold_i8(c, true, m, rows, cols, w, out);
}
int hl_b200_fold_cols_i8(hl_ctx* c, const int8_t* m, size_t rows, size_t cols, const uint64_t* cw, uint64_t* out) {
    return fold_i8(c, false, m, rows, cols, cw, out);
}

}  // extern "C"
