// The masking commitment `M` of a block and the product polynomial of its opening (hashline/src/zk.rs:447-536 mask_commit /
// mask_commit_tagged, :618-656 mask_open): 2 S message rows of 2^log_msg evaluations (a CFS mask's real or imaginary
// coefficients, then its pads, then zeros) and four rows of 2^(log_msg + 1) coefficients (the blinding polynomial b and the
// proximity mask u), every row evaluated on the coset 7 G_dom, columns hashed, leaves salted, tree built.
//
// On the device the commitment is a store (csrc/commit_api.cu) whose data rows are the COEFFICIENT rows, 2^(log_msg + 1)
// words each (a message row's coefficients zero-extended): the column gather, the salted tree and the row fold of a
// store then serve the opening as they are -- the proximity combination sum_row r_row p_row + u (zk.rs:641-647) is the
// store's fold with the weights (r_0 .., 1, U).  What is left is the product polynomial
//   q' = sum_s p_{a_s} p_{W_s} + p_b   (zk.rs:623-637)
// computed here in the evaluation domain of size 2^(log_msg + 1): one CTA per mask transforms a_re, a_im, W_re, W_im and
// writes the two planes of a_s W_s, a last CTA sums them, transforms back once and adds b.  Field arithmetic is exact, so
// the 2^(log_msg + 1) words are the ones the reference's four products per mask give.
#include "api_internal.h"
#include "gl_field.cuh"

using namespace hlapi;

namespace {

struct Tw {
    const u64* tw;  // dom powers of the dom-th root
    u32 logdom;
    __device__ __forceinline__ u64 at(u32 e, u32 logl, bool inv) const {  // w_L^e or w_L^-e, L = 2^logl
        const u32 dom = 1u << logdom, idx = e << (logdom - logl);
        return tw[inv ? (dom - idx) & (dom - 1) : idx];
    }
};

// natural order in, bit-reversed order out
__device__ void ntt_dif(u64* x, u32 logl, const Tw& t, bool inv) {
    const u32 half_n = 1u << (logl - 1);
    for (u32 s = logl; s >= 1; s--) {
        const u32 half = 1u << (s - 1);
        for (u32 p = threadIdx.x; p < half_n; p += blockDim.x) {
            const u32 j = p & (half - 1), i = ((p >> (s - 1)) << s) + j;
            const u64 u = x[i], v = x[i + half];
            x[i] = gl_add(u, v);
            x[i + half] = gl_mul(gl_sub(u, v), t.at(j << (logl - s), logl, inv));
        }
        __syncthreads();
    }
}

// bit-reversed order in, natural order out
__device__ void ntt_dit(u64* x, u32 logl, const Tw& t, bool inv) {
    const u32 half_n = 1u << (logl - 1);
    for (u32 s = 1; s <= logl; s++) {
        const u32 half = 1u << (s - 1);
        for (u32 p = threadIdx.x; p < half_n; p += blockDim.x) {
            const u32 j = p & (half - 1), i = ((p >> (s - 1)) << s) + j;
            const u64 u = x[i], v = gl_mul(x[i + half], t.at(j << (logl - s), logl, inv));
            x[i] = gl_add(u, v);
            x[i + half] = gl_sub(u, v);
        }
        __syncthreads();
    }
}

// CTA s: the two planes of p_{a_s} p_{W_s} at the 2m points of the product domain, bit-reversed order
__global__ void __launch_bounds__(256) k_mask_products(const u64* __restrict__ coefs /* rows of 2m */, const u64* __restrict__ ws /* S x m Fp2 */,
                                                       u32 logm, Tw t, u64 minv, u64* __restrict__ partial /* S x 2 x 2m */) {
    extern __shared__ u64 sm[];
    const u32 m = 1u << logm, m2 = 2 * m, s = blockIdx.x;
    u64 *are = sm, *aim = sm + m2, *wre = sm + 2 * m2, *wim = sm + 3 * m2;
    for (u32 i = threadIdx.x; i < m2; i += blockDim.x) {
        are[i] = coefs[(size_t)(2 * s) * m2 + i];
        aim[i] = coefs[(size_t)(2 * s + 1) * m2 + i];
        wre[i] = 0;
        wim[i] = 0;
    }
    __syncthreads();
    // p_W interpolates W on G_m (zk.rs:596-602): the inverse transform, its input placed in bit-reversed order
    for (u32 i = threadIdx.x; i < m; i += blockDim.x) {
        const u32 r = __brev(i) >> (32 - logm);
        wre[r] = ws[((size_t)s * m + i) * 2];
        wim[r] = ws[((size_t)s * m + i) * 2 + 1];
    }
    __syncthreads();
    ntt_dit(wre, logm, t, true);
    ntt_dit(wim, logm, t, true);
    for (u32 i = threadIdx.x; i < m; i += blockDim.x) {
        wre[i] = gl_mul(wre[i], minv);
        wim[i] = gl_mul(wim[i], minv);
    }
    __syncthreads();
    ntt_dif(are, logm + 1, t, false);
    ntt_dif(aim, logm + 1, t, false);
    ntt_dif(wre, logm + 1, t, false);
    ntt_dif(wim, logm + 1, t, false);
    u64* out = partial + (size_t)s * 2 * m2;
    for (u32 k = threadIdx.x; k < m2; k += blockDim.x) {
        const fp2 p = f2_mul(f2(are[k], aim[k]), f2(wre[k], wim[k]));  // (a_re + U a_im)(W_re + U W_im), U^2 = 7
        out[k] = p.c0;
        out[m2 + k] = p.c1;
    }
}

// one CTA: sum of the S products, back to coefficients, plus b
__global__ void __launch_bounds__(1024) k_mask_q(const u64* __restrict__ partial, u32 S, const u64* __restrict__ b_re, const u64* __restrict__ b_im,
                                                 u32 logm, Tw t, u64 m2inv, u64* __restrict__ q /* 2m Fp2 */) {
    extern __shared__ u64 sm[];
    const u32 m2 = 2u << logm;
    u64 *re = sm, *im = sm + m2;
    for (u32 k = threadIdx.x; k < m2; k += blockDim.x) {
        u64 a = 0, b = 0;
        for (u32 s = 0; s < S; s++) {
            a = gl_add(a, partial[(size_t)s * 2 * m2 + k]);
            b = gl_add(b, partial[(size_t)s * 2 * m2 + m2 + k]);
        }
        re[k] = a;
        im[k] = b;
    }
    __syncthreads();
    ntt_dit(re, logm + 1, t, true);
    ntt_dit(im, logm + 1, t, true);
    for (u32 i = threadIdx.x; i < m2; i += blockDim.x) {
        q[2 * i] = gl_add(gl_mul(re[i], m2inv), b_re[i]);
        q[2 * i + 1] = gl_add(gl_mul(im[i], m2inv), b_im[i]);
    }
}

}  // namespace

extern "C" {

int hl_b200_mask_commit(hl_ctx* c, uint32_t log_msg, uint32_t log_dom, const uint64_t* msgs, size_t n_msg_rows, const uint64_t* coef_rows,
                        size_t n_coef_rows, const uint64_t* pows, const uint8_t* key32, hl_store** store, uint64_t* a_coefs, uint8_t* leaves32) {
    if (!c || !msgs || !coef_rows || !pows || !store || !leaves32) return fail(c, HL_B200_ERR_ARG, "mask_commit: null argument");
    if (log_msg < 8 || log_msg > 11 || log_dom < log_msg + 1 || log_dom > log_msg + 6)
        return fail(c, HL_B200_ERR_UNSUPPORTED, "mask_commit: messages of 2^8 .. 2^11 words, domain 2 .. 64 times the message");
    if (n_msg_rows == 0 || n_msg_rows > 4096 || n_coef_rows == 0 || n_coef_rows > 64) return fail(c, HL_B200_ERR_ARG, "mask_commit: row counts");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    const size_t m = (size_t)1 << log_msg, m2 = 2 * m, dom = (size_t)1 << log_dom, rows = n_msg_rows + n_coef_rows;
    hl_store* st = new hl_store();
    st->ctx = c; st->rows = (u32)rows; st->logn = log_msg + 1; st->logr = log_dom - log_msg - 1; st->q = 0; st->zk = false; st->fold_data = true;
    u64 *d_msgs = nullptr, *d_pows = nullptr, *scratch = nullptr;
    uint32_t* d_key = nullptr;
    const u64* tw = nullptr;
    const size_t scratch_words = hlk::encode_scratch_words(log_msg, 2, c->sm_count, (u32)rows);
    int rc = root_powers(c, log_dom, &tw);
    if (!rc) rc = dev_alloc(c, (void**)&st->d_data, rows * m2 * 8);
    if (!rc) rc = dev_alloc(c, (void**)&st->d_enc, rows * dom * 8);
    if (!rc) rc = dev_alloc(c, (void**)&st->d_leaves, dom * 32);
    if (!rc) rc = dev_alloc(c, (void**)&d_msgs, n_msg_rows * m * 8);
    if (!rc) rc = dev_alloc(c, (void**)&d_pows, dom * 8);
    if (!rc) rc = dev_alloc(c, (void**)&scratch, scratch_words * 8);
    uint32_t* cvs = nullptr;
    const size_t cvs_bytes = hlk::hash_chunks((u32)rows) > 1 ? (size_t)hlk::hash_chunks((u32)rows) * dom * 32 : 0;
    if (!rc && cvs_bytes) rc = dev_alloc(c, (void**)&cvs, cvs_bytes);
    if (!rc) rc = upload_key(c, key32, &d_key);
    if (!rc && cudaMemsetAsync(st->d_data, 0, n_msg_rows * m2 * 8, c->stream) != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "mask_commit: clear");
    if (!rc) rc = h2d(c, d_msgs, msgs, n_msg_rows * m * 8);
    if (!rc) rc = h2d(c, st->d_data + n_msg_rows * m2, coef_rows, n_coef_rows * m2 * 8);
    if (!rc) rc = h2d(c, d_pows, pows, dom * 8);
    if (!rc) {
        Timed t(c, HL_T_ENCODE);
        enc::RowArgs a;
        a.pads = nullptr; a.pows = d_pows; a.tw_nn = tw; a.scratch = scratch; a.loga = 0; a.zk = 0; a.split = 0;
        a.ninv = gl_inv((u64)m);
        // message rows: m evaluations -> coefficients (kept) -> the coset
        a.data = d_msgs; a.enc = st->d_enc; a.rows = (u32)n_msg_rows; a.q = 0; a.T = 1; a.logr = log_dom - log_msg; a.coef_out = st->d_data;
        cudaError_t e = hlk::encode_rows_form(a, log_msg, enc::FORM_COSET, c->sm_count, scratch_words, c->stream);
        // coefficient rows: 2m coefficients -> the coset
        a.data = st->d_data + n_msg_rows * m2; a.enc = st->d_enc + n_msg_rows * dom; a.rows = (u32)n_coef_rows; a.q = (u32)m; a.T = 2; a.coef_out = nullptr;
        if (e == cudaSuccess) e = hlk::encode_rows_form(a, log_msg, enc::FORM_COEF, c->sm_count, scratch_words, c->stream);
        c->stats.kernel_launches += 2;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "mask_commit: row encoder launch", e);
    }
    if (!rc) {
        Timed t(c, HL_T_HASH);
        cudaError_t e = hlk::hash_columns(st->d_enc, st->rows, (u32)dom, d_key, cvs, st->d_leaves, c->stream);
        c->stats.kernel_launches += 1;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "mask_commit: column hash launch", e);
    }
    if (!rc && a_coefs) {
        cudaError_t e = cudaMemcpy2DAsync(a_coefs, m * 8, st->d_data, m2 * 8, m * 8, n_msg_rows, cudaMemcpyDeviceToHost, c->stream);
        c->stats.bytes_d2h += n_msg_rows * m * 8;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "mask_commit: coefficient read", e);
    }
    if (!rc) rc = d2h(c, leaves32, st->d_leaves, dom * 32);
    if (!rc) rc = sync(c, "mask_commit");
    else cudaStreamSynchronize(c->stream);
    dev_free(c, d_msgs, n_msg_rows * m * 8);
    dev_free(c, d_pows, dom * 8);
    dev_free(c, scratch, scratch_words * 8);
    if (d_key) dev_free(c, d_key, 32);
    if (cvs) dev_free(c, cvs, cvs_bytes);
    if (rc) { store_release(st); return rc; }
    c->stats.commits++;
    c->stores.insert(st);
    *store = st;
    return HL_B200_OK;
}

int hl_b200_mask_open_q(hl_store* st, size_t n_masks, const uint64_t* ws, uint64_t* q) {
    if (!st) return HL_B200_ERR_ARG;
    hl_ctx* c = st->ctx;
    if (!ws || !q || n_masks == 0) return fail(c, HL_B200_ERR_ARG, "mask_open_q: null argument");
    if (!st->fold_data || !st->d_data || st->logn < 9 || 2 * n_masks + 2 > st->rows) return fail(c, HL_B200_ERR_ARG, "mask_open_q: not a masking commitment of that many masks");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    const u32 logm = st->logn - 1, logdom = st->logn + st->logr;
    const size_t m = (size_t)1 << logm, m2 = 2 * m;
    const u64* tw = nullptr;
    u64 *d_ws = nullptr, *d_part = nullptr, *d_q = nullptr;
    int rc = root_powers(c, logdom, &tw);
    if (!rc) rc = dev_alloc(c, (void**)&d_ws, n_masks * m * 16);
    if (!rc) rc = dev_alloc(c, (void**)&d_part, n_masks * 2 * m2 * 8);
    if (!rc) rc = dev_alloc(c, (void**)&d_q, m2 * 16);
    if (!rc) rc = h2d(c, d_ws, ws, n_masks * m * 16);
    if (!rc) {
        Timed t(c, HL_T_FOLD);
        const Tw T{tw, logdom};
        const size_t sm1 = 4 * m2 * 8, sm2 = 2 * m2 * 8;
        cudaError_t e = cudaFuncSetAttribute(k_mask_products, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm1);
        if (e == cudaSuccess) {
            k_mask_products<<<(unsigned)n_masks, 256, sm1, c->stream>>>(st->d_data, d_ws, logm, T, gl_inv((u64)m), d_part);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaFuncSetAttribute(k_mask_q, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm2);
        if (e == cudaSuccess) {
            const u64* b_re = st->d_data + 2 * n_masks * m2;
            k_mask_q<<<1, 1024, sm2, c->stream>>>(d_part, (u32)n_masks, b_re, b_re + m2, logm, T, gl_inv((u64)m2), d_q);
            e = cudaGetLastError();
        }
        c->stats.kernel_launches += 2;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "mask_open_q: launch", e);
    }
    if (!rc) rc = d2h(c, q, d_q, m2 * 16);
    if (!rc) rc = sync(c, "mask_open_q");
    else cudaStreamSynchronize(c->stream);
    dev_free(c, d_ws, n_masks * m * 16);
    dev_free(c, d_part, n_masks * 2 * m2 * 8);
    dev_free(c, d_q, m2 * 16);
    return rc;
}

}  // extern "C"
