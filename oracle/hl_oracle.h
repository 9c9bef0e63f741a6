/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * CPU restatement ("oracle") of the reference prover's hot path: Goldilocks
 * field, NTT / Reed-Solomon row encoding, BLAKE3 column leaves, Merkle tree,
 * Fiat-Shamir transcript, prover RNG, multilinear folds, sumcheck with CFS
 * masking, LogUp inverses.  Only tests, the smoke check and the bench's CPU
 * baseline may load it; the product library never does.
 *
 * Each function names the reference source it follows (paths relative to the
 * reference's ops/zkp-mvp/gpu-metal tree).
 */
#ifndef HL_ORACLE_H
#define HL_ORACLE_H
#include "field.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- blake3.c ---- */
void or_blake3(const uint8_t *key, const uint8_t *data, size_t len, uint8_t *out, size_t outlen);
void or_blake3_derive_key(const uint8_t *context, size_t ctx_len, const uint8_t *material, size_t len, uint8_t out[32]);

/* ---- field probes (field.rs) ---- */
uint64_t or_fp_add(uint64_t a, uint64_t b);
uint64_t or_fp_sub(uint64_t a, uint64_t b);
uint64_t or_fp_mul(uint64_t a, uint64_t b);
uint64_t or_fp_neg(uint64_t a);
uint64_t or_fp_inv(uint64_t a);
uint64_t or_fp_pow(uint64_t a, uint64_t e);
uint64_t or_fp_new(uint64_t a);
uint64_t or_fp_from_u128(uint64_t hi, uint64_t lo);
uint64_t or_fp_from_i64(int64_t v);
uint64_t or_two_adic_root(uint32_t k);
void or_fp2_mul(const uint64_t a[2], const uint64_t b[2], uint64_t out[2]);
void or_fp2_inv(const uint64_t a[2], uint64_t out[2]);
void or_batch_inverse2(uint64_t *vals /* n x 2, in place */, size_t n);

/* ---- ntt.c (ntt.rs, pcs.rs, pcs/encode_buffer.rs) ---- */
void or_ntt_forward(uint64_t *a, uint32_t log_n, uint32_t max_log);
void or_ntt_inverse(uint64_t *a, uint32_t log_n, uint32_t max_log);
void or_coset_powers(uint64_t h, size_t nn, uint64_t *out);
void or_encode_row_zk(const uint64_t *msg, size_t n, const uint64_t *pad, size_t q, const uint64_t *pows,
                      size_t nn, uint32_t max_log, uint64_t *out);
void or_encode_rows_zk(const uint64_t *data, size_t rows, size_t n, const uint64_t *pads, size_t q,
                       const uint64_t *pows, size_t nn, uint32_t max_log, uint64_t *encoded);
void or_encode_rows_plain(const uint64_t *data, size_t rows, size_t n, size_t nn, uint32_t max_log, uint64_t *encoded);
void or_hash_columns(const uint64_t *encoded, size_t rows, size_t nn, const uint8_t *key, uint8_t *leaves);
void or_salt_leaves(const uint8_t *leaves, const uint8_t *salts, size_t nn, const uint8_t *leaf_key, uint8_t *out);
/* levels_out: (2*nn - 1) digests: nn salted leaves, nn/2, ..., 1 (the root last) */
void or_merkle_build(const uint8_t *leaves, size_t nn, const uint8_t *node_key, uint8_t *levels_out);
void or_fold_rows(const uint64_t *src, size_t rows, size_t n, size_t nn, size_t ir,
                  const uint64_t *rhos /* k x rows x 2 */, size_t k, uint64_t *out /* k x n x 2 */);
void or_gather_columns(const uint64_t *encoded, size_t rows, size_t nn, const uint64_t *idx, size_t nidx, uint64_t *out);
/* whole hiding commitment: encode, hash columns, salt, tree; returns levels */
void or_commit_zk(const uint64_t *data, size_t rows, size_t n, const uint64_t *pads, size_t q, const uint64_t *pows,
                  size_t nn, uint32_t max_log, const uint8_t *col_key, const uint8_t *salts,
                  const uint8_t *leaf_key, const uint8_t *node_key,
                  uint64_t *encoded, uint8_t *leaves, uint8_t *levels_out);

/* ---- transcript.c (transcript.rs, rng.rs) ---- */
typedef struct { uint8_t state[32]; uint64_t counter; uint8_t key[32]; int keyed; } or_transcript;
void or_tr_new(or_transcript *t, const uint8_t *domain, size_t len, const uint8_t *key);
void or_tr_absorb(or_transcript *t, const uint8_t *label, size_t llen, const uint8_t *data, size_t dlen);
void or_tr_squeeze(or_transcript *t, uint8_t out[32]);
uint64_t or_tr_challenge_fp(or_transcript *t);
void or_tr_challenge_fp2(or_transcript *t, uint64_t out[2]);
void or_tr_challenge_indices(or_transcript *t, size_t n, uint64_t bound, uint64_t *out);

typedef struct { uint8_t key[32]; uint64_t counter; uint8_t buf[8192]; size_t pos; } or_rng;
void or_rng_new(or_rng *r, uint64_t seed, const uint8_t *domain, size_t len);
uint64_t or_rng_next_u64(or_rng *r);
uint64_t or_rng_fp(or_rng *r);
void or_rng_fill_fp(or_rng *r, uint64_t *out, size_t n);
void or_rng_bytes32(or_rng *r, uint8_t out[32]);

/* ---- tables.c (private_block/argument.rs host table builders) ---- */
void or_eq_cube(const uint64_t *point, size_t p, size_t n_vars, size_t start, uint64_t *out);
void or_priv_table(const int32_t *kind, const uint32_t *var, const uint64_t *fixed, size_t log,
                   const uint64_t *slices, size_t ns, const uint64_t *data, size_t n_vars, uint64_t *out);

/* ---- sumcheck.c (mle.rs, sumcheck.rs, sumcheck/rounds.rs) ---- */
void or_eq_table(const uint64_t *r, size_t n, uint64_t *out);
void or_eq_table_msb(const uint64_t *r, size_t n, uint64_t *out);
void or_interpolate_eval(const uint64_t *vals, size_t d, const uint64_t x[2], uint64_t out[2]);
void or_fold_rows_i8(const int8_t *m, size_t rows, size_t cols, const uint64_t *w, uint64_t *out);
void or_fold_cols_i8(const int8_t *m, size_t rows, size_t cols, const uint64_t *c, uint64_t *out);
/* poly ids: 0 = product of all k tables; 1 = t0 * (t1 * t2 - t3);
 * 2 = LogUp query zero-check  t0 * (t1 * (alpha - t2) - 1)        (coefs = alpha)
 * 3 = LogUp table zero-check  t0 * (t1 * (alpha - t2) - t3)       (coefs = alpha)
 * 4 = the slot polynomial last given to or_ir_set (private_block/slot_ir.rs:352-377), coefs = its Fp2 coefficients */
void or_ir_set(const uint32_t *words, size_t n_nodes, size_t n_terms);
void or_poly_eval(int poly, const uint64_t *vals /* k x 2 */, size_t k, const uint64_t *coefs, uint64_t out[2]);
void or_sc_round(int poly, const uint64_t *tables, size_t k, size_t len, size_t degree, const uint64_t *coefs,
                 int eval_one, uint64_t *sums);
void or_sc_fold(uint64_t *tables, size_t k, size_t len, size_t stride, const uint64_t r[2]);
void or_cfs_round(const uint64_t *coeffs, size_t n_vars, size_t degree, size_t j, const uint64_t *prev, uint64_t *out);
void or_cfs_total(const uint64_t *coeffs, size_t n_vars, size_t degree, uint64_t out[2]);
void or_cfs_eval(const uint64_t *coeffs, size_t n_vars, size_t degree, const uint64_t *rho, uint64_t out[2]);
/* whole (optionally masked) sumcheck as prove_rounds drives it; tables folded in place (stride = len).
 * mask == NULL: plain.  out_rounds: n x (degree+1) unmasked, out_masked: same shape (masked messages,
 * equal to out_rounds when plain), out_chal: n, out_finals: k. */
void or_sc_prove(int poly, uint64_t *tables, size_t k, size_t n_vars, size_t degree, const uint64_t *coefs,
                 const uint64_t *mask, const uint64_t mask_c[2], size_t mask_vars, int recover_one,
                 const uint64_t *claim, or_transcript *tr,
                 uint64_t *out_rounds, uint64_t *out_masked, uint64_t *out_chal, uint64_t *out_finals);

/* ---- logup.c (hashline private_block/protocol.rs:993-1007,1125-1140; accuracy_act.rs:13-117) ---- */
void or_logup_histogram(const int32_t *idx, size_t nq, size_t table_len, uint64_t *mult);
void or_logup_helpers(const int32_t *idx, const int32_t *outv, size_t nq, const uint64_t alpha[2],
                      const uint64_t beta[2], const uint64_t gamma_tag[2], int64_t idx_off, uint64_t *h /* nq x 2 */);
void or_logup_table_helper(const int32_t *table_out, const uint64_t *mult, size_t table_len, const uint64_t alpha[2],
                           const uint64_t beta[2], const uint64_t gamma_tag[2], uint64_t *ht /* table_len x 2 */);

void or_logup_query_values(const int32_t *idx, const int32_t *outv, size_t n, const uint64_t beta[2],
                           const uint64_t gamma_tag[2], int64_t idx_off, uint64_t *q);
void or_fp2_sum(const uint64_t *v, size_t n, uint64_t out[2]);

int or_num_threads(void);
void or_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
