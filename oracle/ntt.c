/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * CPU restatement of the reference's NTT, row encoder, column hash, Merkle
 * tree, opening fold and column gather.
 */
#include "hl_oracle.h"
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* the launcher of a multi-process job pins OMP_NUM_THREADS to 1; the CPU baseline wants the host's cores */
void or_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int or_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

uint64_t or_fp_add(uint64_t a, uint64_t b) { return fp_add(a, b); }
uint64_t or_fp_sub(uint64_t a, uint64_t b) { return fp_sub(a, b); }
uint64_t or_fp_mul(uint64_t a, uint64_t b) { return fp_mul(a, b); }
uint64_t or_fp_neg(uint64_t a) { return fp_neg(a); }
uint64_t or_fp_inv(uint64_t a) { return fp_inv(a); }
uint64_t or_fp_pow(uint64_t a, uint64_t e) { return fp_pow(a, e); }
uint64_t or_fp_new(uint64_t a) { return fp_new(a); }
uint64_t or_fp_from_u128(uint64_t hi, uint64_t lo) { return fp_reduce128(((u128)hi << 64) | lo); }
uint64_t or_fp_from_i64(int64_t v) { return fp_from_i64(v); }
uint64_t or_two_adic_root(uint32_t k) { return fp_two_adic_root(k); }
void or_fp2_mul(const uint64_t a[2], const uint64_t b[2], uint64_t out[2]) {
    fp2_t r = fp2_mul(fp2_new(a[0], a[1]), fp2_new(b[0], b[1]));
    out[0] = r.c0; out[1] = r.c1;
}
void or_fp2_inv(const uint64_t a[2], uint64_t out[2]) {
    fp2_t r = fp2_inv(fp2_new(a[0], a[1]));
    out[0] = r.c0; out[1] = r.c1;
}
/* field.rs:212-227: prefix products in index order, one inversion, backward sweep */
void or_batch_inverse2(uint64_t *vals, size_t n) {
    if (!n) return;
    fp2_t *v = (fp2_t *)vals;
    fp2_t *prefix = (fp2_t *)malloc(n * sizeof(fp2_t));
    fp2_t acc = FP2_ONE;
    for (size_t i = 0; i < n; i++) { prefix[i] = acc; acc = fp2_mul(acc, v[i]); }
    fp2_t inv = fp2_inv(acc);
    for (size_t i = n; i-- > 0;) {
        fp2_t x = v[i];
        v[i] = fp2_mul(inv, prefix[i]);
        inv = fp2_mul(inv, x);
    }
    free(prefix);
}

/* ntt.rs:29-43: one shared table of 2^(max_log-1) powers of the 2^max_log-th
 * root, forward and inverse; a size-len stage reads tw[k * (max_n / len)]. */
typedef struct { uint32_t max_log; uint64_t *fwd, *inv; } tables_t;
static tables_t g_tabs[40];

static const tables_t *tables_for(uint32_t max_log) {
    tables_t *t = &g_tabs[max_log];
    if (t->fwd) return t;
#pragma omp critical(or_tables)
    {
        if (!t->fwd) {
            size_t half = (size_t)1 << (max_log ? max_log - 1 : 0);
            uint64_t *f = (uint64_t *)malloc(half * 8), *iv = (uint64_t *)malloc(half * 8);
            uint64_t w = fp_two_adic_root(max_log), wi = fp_inv(w), c = 1, ci = 1;
            for (size_t i = 0; i < half; i++) { f[i] = c; iv[i] = ci; c = fp_mul(c, w); ci = fp_mul(ci, wi); }
            t->inv = iv; t->max_log = max_log;
            __atomic_store_n(&t->fwd, f, __ATOMIC_RELEASE);
        }
    }
    return t;
}

/* ntt.rs:69-108: bit-reverse the input in place, then decimation-in-time
 * stages len = 2, 4, ..., n; output in natural order. */
static void transform(uint64_t *a, uint32_t log_n, const uint64_t *tw, uint32_t max_log) {
    size_t n = (size_t)1 << log_n;
    if (n == 1) return;
    size_t j = 0;
    for (size_t i = 1; i < n; i++) {
        size_t bit = n >> 1;
        while (j & bit) { j ^= bit; bit >>= 1; }
        j |= bit;
        if (i < j) { uint64_t t = a[i]; a[i] = a[j]; a[j] = t; }
    }
    size_t max_n = (size_t)1 << max_log;
    for (size_t len = 2; len <= n; len <<= 1) {
        size_t half = len / 2, stride = max_n / len;
        for (size_t i = 0; i < n; i += len)
            for (size_t k = 0; k < half; k++) {
                uint64_t u = a[i + k], v = fp_mul(a[i + k + half], tw[k * stride]);
                a[i + k] = fp_add(u, v);
                a[i + k + half] = fp_sub(u, v);
            }
    }
}

void or_ntt_forward(uint64_t *a, uint32_t log_n, uint32_t max_log) {
    transform(a, log_n, tables_for(max_log)->fwd, max_log);
}
/* ntt.rs:60-67: inverse-table transform, then every entry times n^-1 */
void or_ntt_inverse(uint64_t *a, uint32_t log_n, uint32_t max_log) {
    transform(a, log_n, tables_for(max_log)->inv, max_log);
    uint64_t ninv = fp_inv(fp_new((uint64_t)1 << log_n));
    for (size_t i = 0; i < ((size_t)1 << log_n); i++) a[i] = fp_mul(a[i], ninv);
}

/* pcs.rs:661-670 */
void or_coset_powers(uint64_t h, size_t nn, uint64_t *out) {
    uint64_t x = 1;
    for (size_t i = 0; i < nn; i++) { out[i] = x; x = fp_mul(x, h); }
}

static uint32_t log2z(size_t n) { uint32_t l = 0; while (((size_t)1 << l) < n) l++; return l; }

/* pcs.rs:674-693 (encode_row_zk); the q > n interleaving is that of
 * pcs/encode_buffer.rs:56-64 and falls out of the in-order loop below. */
void or_encode_row_zk(const uint64_t *msg, size_t n, const uint64_t *pad, size_t q, const uint64_t *pows,
                      size_t nn, uint32_t max_log, uint64_t *out) {
    memcpy(out, msg, n * 8);
    or_ntt_inverse(out, log2z(n), max_log);
    memset(out + n, 0, (nn - n) * 8);
    for (size_t i = 0; i < q; i++) { out[i] = fp_sub(out[i], pad[i]); out[n + i] = pad[i]; }
    for (size_t i = 0; i < n + q; i++) out[i] = fp_mul(out[i], pows[i]);
    or_ntt_forward(out, log2z(nn), max_log);
}

/* pcs.rs:752-754 / encode_buffer.rs:10-41: rows are independent tasks */
void or_encode_rows_zk(const uint64_t *data, size_t rows, size_t n, const uint64_t *pads, size_t q,
                       const uint64_t *pows, size_t nn, uint32_t max_log, uint64_t *encoded) {
    tables_for(max_log);
#pragma omp parallel for schedule(dynamic, 1)
    for (size_t r = 0; r < rows; r++)
        or_encode_row_zk(data + r * n, n, pads + r * q, q, pows, nn, max_log, encoded + r * nn);
}

/* pcs.rs:241-246 with ntt.rs:113-122: systematic Reed-Solomon rows */
void or_encode_rows_plain(const uint64_t *data, size_t rows, size_t n, size_t nn, uint32_t max_log, uint64_t *encoded) {
    tables_for(max_log);
#pragma omp parallel for schedule(dynamic, 1)
    for (size_t r = 0; r < rows; r++) {
        uint64_t *e = encoded + r * nn;
        memcpy(e, data + r * n, n * 8);
        or_ntt_inverse(e, log2z(n), max_log);
        memset(e + n, 0, (nn - n) * 8);
        or_ntt_forward(e, log2z(nn), max_log);
    }
}

/* pcs.rs:176-221: leaf j = BLAKE3[keyed] of column j's words, row 0 first,
 * 8 little-endian bytes each; tiles of 64 columns per task. */
void or_hash_columns(const uint64_t *encoded, size_t rows, size_t nn, const uint8_t *key, uint8_t *leaves) {
    const size_t tile = 64;
    size_t ntiles = (nn + tile - 1) / tile;
#pragma omp parallel
    {
        uint64_t *buf = (uint64_t *)malloc(tile * rows * 8);
#pragma omp for schedule(dynamic, 1)
        for (size_t t = 0; t < ntiles; t++) {
            size_t c0 = t * tile, w = nn - c0 < tile ? nn - c0 : tile;
            for (size_t i = 0; i < rows; i++)
                for (size_t c = 0; c < w; c++) buf[c * rows + i] = encoded[i * nn + c0 + c];
            for (size_t c = 0; c < w; c++)
                or_blake3(key, (const uint8_t *)(buf + c * rows), rows * 8, leaves + 32 * (c0 + c), 32);
        }
        free(buf);
    }
}

/* pcs.rs:696-715: salted = H_leaf(leaf || salt) */
void or_salt_leaves(const uint8_t *leaves, const uint8_t *salts, size_t nn, const uint8_t *leaf_key, uint8_t *out) {
#pragma omp parallel for
    for (size_t j = 0; j < nn; j++) {
        uint8_t m[64];
        memcpy(m, leaves + 32 * j, 32);
        memcpy(m + 32, salts + 32 * j, 32);
        or_blake3(leaf_key, m, 64, out + 32 * j, 32);
    }
}

/* merkle.rs:48-81: node = H_node(left || right); levels halve down to the root */
void or_merkle_build(const uint8_t *leaves, size_t nn, const uint8_t *node_key, uint8_t *levels_out) {
    memcpy(levels_out, leaves, nn * 32);
    const uint8_t *prev = levels_out;
    uint8_t *next = levels_out + nn * 32;
    for (size_t w = nn / 2; w >= 1; w /= 2) {
#pragma omp parallel for if (w >= 1024)
        for (size_t i = 0; i < w; i++) or_blake3(node_key, prev + 64 * i, 64, next + 32 * i, 32);
        prev = next;
        next += w * 32;
        if (w == 1) break;
    }
}

/* pcs.rs:342-378 (fold_rows_host): out[g][j] = sum_i rho_g[i] * src[i*nn + j*ir];
 * the zero skips there only save work, the sums are exact field sums. */
void or_fold_rows(const uint64_t *src, size_t rows, size_t n, size_t nn, size_t ir,
                  const uint64_t *rhos, size_t k, uint64_t *out) {
    const fp2_t *rho = (const fp2_t *)rhos;
    fp2_t *o = (fp2_t *)out;
    size_t chunk = n < 512 ? n : 512, nch = (n + chunk - 1) / chunk;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (size_t g = 0; g < k; g++)
        for (size_t ci = 0; ci < nch; ci++) {
            size_t c0 = ci * chunk, w = n - c0 < chunk ? n - c0 : chunk;
            fp2_t acc[512];
            for (size_t j = 0; j < w; j++) acc[j] = FP2_ZERO;
            for (size_t i = 0; i < rows; i++) {
                fp2_t r = rho[g * rows + i];
                if (fp2_is_zero(r)) continue;
                const uint64_t *row = src + i * nn;
                for (size_t j = 0; j < w; j++) {
                    uint64_t v = row[(c0 + j) * ir];
                    if (v) acc[j] = fp2_add(acc[j], fp2_mul_base(r, v));
                }
            }
            for (size_t j = 0; j < w; j++) o[g * n + c0 + j] = acc[j];
        }
}

/* pcs.rs:1055-1067: column idx[c] of the encoded matrix, rows entries, idx order */
void or_gather_columns(const uint64_t *encoded, size_t rows, size_t nn, const uint64_t *idx, size_t nidx, uint64_t *out) {
    for (size_t c = 0; c < nidx; c++)
        for (size_t i = 0; i < rows; i++) out[c * rows + i] = encoded[i * nn + idx[c]];
}

/* pcs.rs:782-817 (commit_zk_owned_with_tag) after the pads and salts are drawn */
void or_commit_zk(const uint64_t *data, size_t rows, size_t n, const uint64_t *pads, size_t q, const uint64_t *pows,
                  size_t nn, uint32_t max_log, const uint8_t *col_key, const uint8_t *salts,
                  const uint8_t *leaf_key, const uint8_t *node_key,
                  uint64_t *encoded, uint8_t *leaves, uint8_t *levels_out) {
    or_encode_rows_zk(data, rows, n, pads, q, pows, nn, max_log, encoded);
    or_hash_columns(encoded, rows, nn, col_key, leaves);
    uint8_t *salted = (uint8_t *)malloc(nn * 32);
    or_salt_leaves(leaves, salts, nn, leaf_key, salted);
    or_merkle_build(salted, nn, node_key, levels_out);
    free(salted);
}
