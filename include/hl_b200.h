/*
 * hl_b200 - the B200 (sm_100a) backend of the Hashline prover's data-parallel hot path,
 * as a C-ABI shared library.
 *
 * The reference prover (Rust) reaches an accelerator through two seams:
 *   zkp-core/src/pcs/backend.rs:30-100      trait EncodedStore, trait Backend
 *   zkp-core/src/sumcheck/rounds.rs:22-28   trait SumcheckRounds
 * and the adapter in hashline/src/gpu/mod.rs:687-859 plugs a device into them.  Every
 * entry point below is what an `impl Backend / EncodedStore / SumcheckRounds` for this
 * backend binds over FFI; each comment names the reference item it stands for.
 * (paths are relative to the reference's ops/zkp-mvp/gpu-metal tree)
 *
 * Conventions
 *  - Field elements are canonical Goldilocks words (uint64_t < p, p = 2^64 - 2^32 + 1);
 *    an Fp2 is two consecutive words (c0, c1) (field.rs:139-203).  Digests are 32 bytes.
 *  - Every pointer is HOST memory unless its name starts with d_.  Inputs are read during
 *    the call only; outputs are complete when the call returns (the *_dev calls are
 *    asynchronous on the context's stream and say so).
 *  - Every call returns 0 (HL_B200_OK) or a negative HL_B200_ERR_*; hl_b200_last_error
 *    gives the text.  A non-zero status is the seam's "decline" (backend.rs:66-71); there
 *    is no CPU fallback inside the library and nothing aborts.
 *  - Results are the reference CPU backend's bytes: the library draws no randomness and
 *    touches no transcript except the replayable round batch of hl_b200_rounds_batched.
 *  - A context serialises its calls with a mutex; use one context per host thread for
 *    concurrent forks (run_fork.rs:1677-1779).
 */
#ifndef HL_B200_H
#define HL_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct hl_ctx hl_ctx;
typedef struct hl_store hl_store;
typedef struct hl_rounds hl_rounds;

enum {
    HL_B200_OK = 0,
    HL_B200_ERR_ARG = -1,         /* a shape or pointer the call cannot take */
    HL_B200_ERR_OOM = -2,         /* device allocation failed */
    HL_B200_ERR_DEVICE = -3,      /* a CUDA call failed; see hl_b200_last_error */
    HL_B200_ERR_TIMEOUT = -4,     /* a bounded device wait ran out */
    HL_B200_ERR_MISMATCH = -5,    /* a self-check failed */
    HL_B200_ERR_ZERO = -6,        /* zero denominator or zero challenge: "discard attempt" (protocol.rs:1059) */
    HL_B200_ERR_UNSUPPORTED = -7  /* a size outside the kernels' range; the caller keeps its own path */
};

/* ---- context: hashline/src/gpu/mod.rs:25-58 (enabled, label), metal.rs:75-95 (lazy context) ---- */
int hl_b200_init(int device, hl_ctx** out);
void hl_b200_shutdown(hl_ctx* ctx);
const char* hl_b200_label(hl_ctx* ctx);
const char* hl_b200_last_error(hl_ctx* ctx);
/* Run the context's work on the caller's CUDA stream (a cudaStream_t); NULL restores its own. */
int hl_b200_set_stream(hl_ctx* ctx, void* cuda_stream);
int hl_b200_sync(hl_ctx* ctx);
/* Failure injection on the HOST side (hashline/src/gpu/mod.rs:121 set_alloc_cap_for_test): with a cap, a device
 * allocation that would bring the context's live bytes above `bytes` fails with HL_B200_ERR_OOM before the
 * runtime is asked; 0 removes the cap.  Nothing on the device is made to fault. */
int hl_b200_set_alloc_cap(hl_ctx* ctx, size_t bytes);
/* Which encoder runs: 0 = radix-2 shared-memory stages (any n <= 2^14), 1 = the 16-point
 * register passes when 2^8 <= n <= 2^14 (default).  Same words either way. */
int hl_b200_set_encoder(hl_ctx* ctx, int fast);
/* Which evaluator runs a slot program whose graph the library has a generated kernel for (the CUDA counterpart of the
 * reference's generated Metal slot kernels, private_block/metal_slot.rs:115-497): 0 = the interpreter, which runs every
 * program (default: it is the faster one on this GPU for every recorded graph), 1 = the generated kernel.  Same words either
 * way; an A/B switch like the reference's HL_GPU_* switches (hashline/src/gpu/cuda.rs:74-125). */
int hl_b200_set_slot_kernels(hl_ctx* ctx, int on);

/* ---- field self-test: metal_probe_field (tests/zk60_metal_commit.rs:69-89), k_probe ----
 * out3n[3i..3i+2] = (a_i + b_i, a_i - b_i, a_i * b_i) */
int hl_b200_probe_field(hl_ctx* ctx, const uint64_t* a, const uint64_t* b, size_t n, uint64_t* out3n);

/* ---- Backend::try_commit (pcs/backend.rs:79-82; CPU body pcs.rs:230-250) ----
 * data: rows x 2^log_cols.  Systematic Reed-Solomon rows to nn = inv_rate 2^log_cols columns,
 * column leaves (unkeyed BLAKE3 when key32 is NULL) into leaves32 (nn x 32 bytes).
 * max_log is the caller's NttTables::max_log (ntt.rs:9-43); it must cover log2 nn and does
 * not change any value.  The store keeps the encoding resident until hl_b200_store_free. */
int hl_b200_commit(hl_ctx* ctx, uint32_t log_cols, uint32_t inv_rate, const uint64_t* data, size_t rows,
                   uint32_t max_log, const uint8_t* key32, hl_store** store, uint8_t* leaves32);

/* ---- Backend::try_commit_zk / try_commit_zk_keyed (pcs/backend.rs:84-99; CPU body
 * pcs.rs:674-693, 782-817 and pcs/encode_buffer.rs:10-71) ----
 * pads: rows x q, pows: nn coset powers.  Returns the UNSALTED leaves; the caller salts and
 * builds the tree (or calls hl_b200_merkle).  The store keeps data, pads and encoding. */
int hl_b200_commit_zk(hl_ctx* ctx, uint32_t log_cols, uint32_t inv_rate, const uint64_t* data, size_t rows,
                      const uint64_t* pads, size_t q, const uint64_t* pows, uint32_t max_log, const uint8_t* key32,
                      hl_store** store, uint8_t* leaves32);

/* hl_b200_commit_zk and hl_b200_store_merkle in one call: commit_zk_owned_with_tag (pcs.rs:782-817) has drawn the salts before it
 * offers the commitment, so they travel with the rows, the salted tree follows the column hash on the device, and leaves32
 * (nn x 32, unsalted; may be NULL: the salted leaves are the first nn entries of levels_out) and levels_out ((2 nn - 1) x 32) come
 * back under one synchronisation. */
int hl_b200_commit_zk_tree(hl_ctx* ctx, uint32_t log_cols, uint32_t inv_rate, const uint64_t* data, size_t rows, const uint64_t* pads, size_t q,
                           const uint64_t* pows, uint32_t max_log, const uint8_t* key32, const uint8_t* salts32, const uint8_t* leaf_key32,
                           const uint8_t* node_key32, hl_store** store, uint8_t* leaves32, uint8_t* levels_out);

/* The hiding commitment from NARROW witness rows: the reference's CUDA uploader sends int8 / int16 / int32 witness planes as 1, 2
 * or 4 bytes per word and restores the identical 64-bit image on the device (hashline/src/gpu/cuda.rs:893-1099 `narrow_class`,
 * `pack_narrow`, `upload_narrow`; kernel `k_widen`, hashline/src/gpu/kernels.cu:220-236; rationale gpu/mod.rs:270-300).
 * packed: the rows back to back, row r as 2^log_cols little-endian two's-complement integers of row_width[r] bytes (1, 2 or 4;
 * a word x >= 0 stands for x, x < 0 for p + x, field.rs:32-34) or, at width 8, its canonical field words as they are.  The
 * width is per ROW here (the reference picks one per upload), so wide rows (masks, hashes) and narrow planes share a call.
 * The bytes are copied as they are and widened inside the encoder's first pass, which also leaves the 64-bit rows resident
 * for the opening.  Every result (leaves, tree, folds, columns) is that of hl_b200_commit_zk[_tree] on the widened matrix.
 * salts32 NULL: no tree (levels_out ignored, leaves32 required); otherwise as hl_b200_commit_zk_tree (leaves32 may be NULL). */
int hl_b200_commit_zk_packed(hl_ctx* ctx, uint32_t log_cols, uint32_t inv_rate, const void* packed, const uint8_t* row_width, size_t rows,
                             const uint64_t* pads, size_t q, const uint64_t* pows, uint32_t max_log, const uint8_t* key32,
                             const uint8_t* salts32, const uint8_t* leaf_key32, const uint8_t* node_key32, hl_store** store,
                             uint8_t* leaves32, uint8_t* levels_out);

/* The same commitment for inputs that already live in device memory (the reference's
 * device-buffer commitment, pcs.rs:801-803 / metal.rs:3105 resident rows).  Asynchronous on
 * the context's stream; d_leaves32 (nn x 32 bytes, device) is ready when the stream reaches
 * this point.  The store BORROWS d_data and d_pads: keep them alive until it is freed. */
int hl_b200_commit_zk_dev(hl_ctx* ctx, uint32_t log_cols, uint32_t inv_rate, const uint64_t* d_data, size_t rows,
                          const uint64_t* d_pads, size_t q, const uint64_t* d_pows, const uint8_t* key32,
                          hl_store** store, uint8_t* d_leaves32);

/* ---- salt_leaf_keyed + MerkleTree::build_keyed (pcs.rs:696-715, merkle.rs:48-81) ----
 * levels_out: (2 nn - 1) x 32 bytes: the nn salted leaves, then each level up, the root last.
 * salts32 NULL: the leaves are used as level 0 unchanged (the plain commitment's tree). */
int hl_b200_merkle(hl_ctx* ctx, const uint8_t* leaves32, const uint8_t* salts32, size_t nn, const uint8_t* leaf_key32,
                   const uint8_t* node_key32, uint8_t* levels_out);
/* The same on the leaves a commit left on the device (no leaf round trip). */
int hl_b200_store_merkle(hl_store* store, const uint8_t* salts32, const uint8_t* leaf_key32, const uint8_t* node_key32,
                         uint8_t* levels_out);

/* The same, device to device and asynchronous on the context's stream: d_salts32 (nn x 32 bytes, or
 * NULL) and d_levels_out ((2 nn - 1) x 32 bytes) are device memory; the root is the last 32 bytes. */
int hl_b200_store_merkle_dev(hl_store* store, const uint8_t* d_salts32, const uint8_t* leaf_key32, const uint8_t* node_key32,
                             uint8_t* d_levels_out);

/* ---- no counterpart in the reference: the column-leaf hash for callers that cannot allocate ----
 * Some callers hold device buffers but may not allocate device memory themselves: a serving loop
 * whose memory was reserved up front, a plug-in inside a process that owns the CUDA pools, a prover
 * thread whose allocation cap is spent.  This call hashes the columns of a rows x nn row-major matrix
 * that is already on the device (d_encoded) into nn 32-byte leaves (d_leaves32, device), keyed when
 * key32 (host) is not NULL, exactly as the commitment's column hash does, and allocates nothing: its
 * scratch (one 32-byte chaining value per column and 128-row chunk) lives in a 24 MiB array inside the
 * library, held by every GPU that loads the library until the process exits.
 * Limits: ceil(rows / 128) * nn * 32 bytes must fit in 24 MiB, else HL_B200_ERR_UNSUPPORTED.
 * It works on the CURRENT device and launches on cuda_stream (a cudaStream_t, NULL = default stream)
 * without waiting for it.  The first call on a device resolves the array's address
 * (cudaGetSymbolAddress); make that call before any stream capture.  Every call on a device shares the
 * array, which keeps the previous call's contents (none of it needs clearing: each call overwrites what
 * it reads); calls that overlap on one GPU race on it and must be serialised by the caller. */
int hl_b200_hash_columns_static(const uint64_t* d_encoded, size_t rows, size_t nn, const uint8_t* key32,
                                uint8_t* d_leaves32, void* cuda_stream);

/* ---- EncodedStore::fold_rows / fold_rows_with_pads (pcs/backend.rs:33-59; CPU body
 * pcs.rs:342-378, 976-1000) ----
 * rhos: k x rows Fp2.  out: k vectors of n Fp2 (with_pads == 0) or n + q Fp2 (with_pads != 0,
 * hiding stores only: the n message entries then rho^T pads). */
int hl_b200_store_fold(hl_store* store, const uint64_t* rhos, size_t k, int with_pads, uint64_t* out);
/* ---- EncodedStore::columns (pcs/backend.rs:37-39; pcs.rs:1055-1067) ----
 * out: nidx x rows words, in the order of idx, duplicates repeated. */
int hl_b200_store_columns(hl_store* store, const uint64_t* idx, size_t nidx, uint64_t* out);
/* rows, n, nn, q of a store (q = 0 for the plain form) */
int hl_b200_store_shape(hl_store* store, size_t* rows, size_t* n, size_t* nn, size_t* q);
/* device address of the encoding (rows x nn words) and of the leaves; for device-side callers */
const uint64_t* hl_b200_store_encoded_dev(hl_store* store);
const uint8_t* hl_b200_store_leaves_dev(hl_store* store);
void hl_b200_store_free(hl_store* store);

/* ---- the verifier's per-column checks of a hiding opening (pcs.rs:1303-1331, the parallel map of `verify_zk_tagged`;
 * merkle.rs:120-127 `verify_path_keyed`; pcs.rs:696-715 `salt_leaf_keyed`) ----
 * cols: ncols runs of `rows` words (OpeningZk::columns in order); idx: the sampled position of each; salts32: ncols x 32;
 * paths32: ncols x depth x 32, the sibling next to the leaf first (the caller has checked every path's length against the
 * tree's depth, pcs.rs:1258-1263); the three keys are NULL for the untagged profile.
 * rhos: k x rows Fp2, the combined row weights of the groups followed by the proximity weights.  What each combination
 * rho_g^T col must equal is given either as `wants` (k x ncols Fp2: the encoded clear vector g at idx[c]) or as
 * `vec_store`, a hiding commitment of the 2k rows (re of vector 0, im of vector 0, re of vector 1, ..) made on this
 * context with store != 0, whose encoding is then read in place.  Exactly one of the two when k > 0.
 * verdict[c]: 0 every check holds; 1 the Merkle path of column c fails; 2 + g column c disagrees with clear vector g
 * (the first such g; the path is checked first, as in the reference).  first_bad (may be NULL): the first c with a
 * non-zero verdict, or -1. */
int hl_b200_verify_columns(hl_ctx* ctx, const uint64_t* cols, size_t rows, size_t ncols, const uint64_t* idx, const uint8_t* salts32,
                           const uint8_t* paths32, uint32_t depth, const uint8_t* root32, const uint8_t* column_key32,
                           const uint8_t* leaf_key32, const uint8_t* node_key32, const uint64_t* rhos, size_t k, const uint64_t* wants,
                           const hl_store* vec_store, int32_t* verdict, int64_t* first_bad);

/* The same with the clear vectors handed over as the opening holds them (pcs.rs:1282-1331 in one call): vecs = k vectors of
 * n + q Fp2 (the group vectors, then the proximity vector); they are split into their 2k real / imaginary rows and encoded on
 * the device by the commitment's encoder (pows = the coset powers of the commitment, nn words), and every column's combinations are
 * compared with that encoding at idx[c].  rhos: k x rows Fp2.  The other arguments and the verdicts are hl_b200_verify_columns'. */
int hl_b200_verify_opening(hl_ctx* ctx, uint32_t log_cols, uint32_t inv_rate, size_t q, const uint64_t* pows, const uint64_t* vecs, size_t k,
                           const uint64_t* cols, size_t rows, size_t ncols, const uint64_t* idx, const uint8_t* salts32,
                           const uint8_t* paths32, uint32_t depth, const uint8_t* root32, const uint8_t* column_key32,
                           const uint8_t* leaf_key32, const uint8_t* node_key32, const uint64_t* rhos, int32_t* verdict, int64_t* first_bad);

/* ---- SumcheckRounds (sumcheck/rounds.rs:22-28; CPU evaluator ClosureRounds :52-167) ----
 * k tables of 2^n_vars Fp2 (table-major, variable 0 = most significant index bit) and a slot polynomial
 * from a fixed family; round j returns the UNMASKED values at 0..=degree of
 * sum_i poly(T(i) + d (T(i + half) - T(i))), fold applies T[i] += r (T[i + half] - T[i]).
 *   HL_POLY_PROD     product of the k tables, degree = k <= 6 (matmul slots v0*v1: argument.rs:2174-2203)
 *   HL_POLY_ZC       t0 * (t1 * t2 - t3), k = 4, degree 3 (zero-check with an eq table)
 *   HL_POLY_LOGUP_Q  t0 * (t1 * (alpha - t2) - 1), k = 3, degree 3, coefs[0] = alpha (LogUp helper constraint)
 *   HL_POLY_LOGUP_T  t0 * (t1 * (alpha - t2) - t3), k = 4, degree 3 (table helper, layout.rs slot 19) */
enum { HL_POLY_PROD = 0, HL_POLY_ZC = 1, HL_POLY_LOGUP_Q = 2, HL_POLY_LOGUP_T = 3 };
int hl_b200_rounds_new(hl_ctx* ctx, int poly, size_t k, uint32_t n_vars, uint32_t degree, const uint64_t* tables,
                       const uint64_t* coefs, size_t ncoefs, hl_rounds** out);
/* The same evaluator for ANY slot polynomial, given as data: the expression graph of
 * private_block/slot_ir.rs:57-345 (tables, affine and sum nodes, top-level terms), which the reference turns
 * into a generated Metal kernel per slot (metal_slot.rs, metal.rs:2627 metal_rounds); here one kernel interprets it.
 * The value at a cube point is that of the reference's interpreter (slot_ir.rs:352-377).
 * `words` (32-bit) = the node records in order, then the term records:
 *     affine node   [0 | count << 8] [konst coef] count x ([coef] [table id])     konst + sum coef_i * table_i
 *     sum node      [1 | count << 8] count x ([coef] [nf] nf x [factor])          sum coef * prod(factors)
 *     term          [coef] [nf] nf x [factor]                                     wrapper tables, then inner factors
 *     factor        table id, or 0x80000000 | node id (a node refers only to earlier nodes)
 *     coef          index into `coefs` (Fp2 each), or HL_IR_ONE / HL_IR_NEG_ONE / HL_IR_ZERO
 * Limits: k <= 64 tables, 128 nodes, 4096 words, 512 coefficients, degree <= 7.  A malformed stream is
 * HL_B200_ERR_ARG and reaches no kernel.  `degree` is the slot's DECLARED degree (the message length); where the
 * graph attains less, the values above the attained degree are extrapolated exactly (gpu/metal.rs:2516-2548). */
#define HL_IR_NODE 0x80000000u
#define HL_IR_ONE 0xFFFFFFFFu
#define HL_IR_NEG_ONE 0xFFFFFFFEu
#define HL_IR_ZERO 0xFFFFFFFDu
int hl_b200_rounds_new_ir(hl_ctx* ctx, size_t k, uint32_t n_vars, uint32_t degree, const uint64_t* tables, const uint32_t* words,
                          size_t n_words, uint32_t n_nodes, uint32_t n_terms, const uint64_t* coefs, size_t ncoefs, hl_rounds** out);
/* ---- the prover's random stream expanded on the device (zkp-core/src/rng.rs:279-417 ZkRng) ----
 * key32 = the generator's key, BLAKE3("hashline-zk-rng/" || domain || LE64(seed)) (rng.rs:280-284), computed by the caller;
 * first_word = u64 words of the stream already consumed; count words (as_fp == 0: next_u64 draws, four per bytes32), or
 * count field elements (as_fp != 0: fp() draws, two words each, rng.rs:323-332).  The caller's generator then skips
 * count (or 2 count) words.  rng_fill writes host memory, rng_fill_dev device memory (e.g. the pads and salts that
 * hl_b200_commit_zk_dev / hl_b200_store_merkle_dev take, in the draw order of pcs.rs:733-745: pads first, then salts). */
int hl_b200_rng_fill(hl_ctx* ctx, const uint8_t* key32, uint64_t first_word, uint64_t count, int as_fp, uint64_t* out);
int hl_b200_rng_fill_dev(hl_ctx* ctx, const uint8_t* key32, uint64_t first_word, uint64_t count, int as_fp, uint64_t* d_out);

/* ---- a slot's tables built on the device (argument.rs:907 build_tables_device; the Metal form is
 * gpu/metal.rs MetalTables::{new, tables_mut, plan_eq, plan_plane, build_planned, flush, to_vecs}) ----
 * A table set is k tables of 2^n_vars Fp2 in device memory.  Each table is filled by ONE of:
 *   tables_put     host-built words (public tables), as MetalTables::tables_mut + flush;
 *   tables_eq      the eq cube of a point over cube variables [start, start + p): entry x is
 *                  hi[y >> p/2] * lo[y & (2^(p/2) - 1)], y = (x >> (n_vars - start - p)) & (2^p - 1), with hi / lo the
 *                  eq tables (msb first) of the point's first p - p/2 and last p/2 coordinates (argument.rs:643-660);
 *   tables_plane   a committed plane: out[x] = sum_z eqf[z] * v(inv_hi[xu >> xlo] | inv_lo[xu & (2^xlo - 1)] | zbits[z]),
 *                  xu = x & used, v(idx) = sum_s coef_s * rows[off_s + idx]; nz = 0 means no fixed coordinate
 *                  (out[x] = v(..)).  The maps are the host builder's own (argument.rs:418-437, 486-512);
 *                  slices = ns x (offset, coef c0, coef c1).  rows = the resident data rows of `store`
 *                  (metal.rs:3105 resident_rows) or, with store NULL, n_words words at the DEVICE address d_rows.
 *                  Every address the maps can form is checked against the rows before the launch.
 * base_check != 0 declares the table base-valued; tables_flush (and rounds_from_tables) answer
 * HL_B200_ERR_MISMATCH if a word of such a table has a non-zero imaginary part (metal.rs:2649-2665).
 * tables_eq and tables_plane PLAN a table (MetalTables::plan_eq / plan_plane): the maps are copied during the call, and every planned
 * table is written by one launch when the set is flushed, read or handed to an evaluator.  The commitment (or the device rows) a
 * planned plane reads must still be there then; a freed store is refused at that point (HL_B200_ERR_ARG), nothing is launched.
 * rounds_from_tables[_ir] takes the set over on success (the handle stays valid but empty; free it). */
typedef struct hl_tables hl_tables;
int hl_b200_tables_new(hl_ctx* ctx, size_t k, uint32_t n_vars, hl_tables** out);
int hl_b200_tables_put(hl_tables* t, size_t i, const uint64_t* words);
int hl_b200_tables_eq(hl_tables* t, size_t i, uint32_t start, uint32_t p, const uint64_t* hi, const uint64_t* lo, int base_check);
int hl_b200_tables_plane(hl_tables* t, size_t i, const hl_store* store, const uint64_t* d_rows, size_t n_words, uint64_t used,
                         uint32_t xlo, const uint32_t* inv_lo, const uint32_t* inv_hi, const uint32_t* zbits, uint32_t nz,
                         const uint64_t* eqf, const uint64_t* slices, uint32_t ns, int base_check);
int hl_b200_tables_flush(hl_tables* t);
int hl_b200_tables_read(hl_tables* t, size_t i, uint64_t* out);   /* MetalTables::to_vecs, one table */
void hl_b200_tables_free(hl_tables* t);
int hl_b200_rounds_from_tables(hl_ctx* ctx, int poly, uint32_t degree, hl_tables* t, const uint64_t* coefs, size_t ncoefs, hl_rounds** out);
int hl_b200_rounds_from_tables_ir(hl_ctx* ctx, uint32_t degree, hl_tables* t, const uint32_t* words, size_t n_words, uint32_t n_nodes,
                                  uint32_t n_terms, const uint64_t* coefs, size_t ncoefs, hl_rounds** out);
/* SumcheckRounds::round: sums = degree + 1 Fp2.  eval_one == 0 skips the point 1 (left zero): the caller
 * recovers s(1) = claim - s(0) (rounds.rs:94-99,137-140). */
int hl_b200_rounds_round(hl_rounds* r, uint32_t j, int eval_one, uint64_t* sums);
/* SumcheckRounds::fold */
int hl_b200_rounds_fold(hl_rounds* r, const uint64_t challenge[2]);
/* SumcheckRounds::finals: k Fp2, the caller's table order */
int hl_b200_rounds_finals(hl_rounds* r, uint64_t* out);
void hl_b200_rounds_free(hl_rounds* r);

/* The transcript position a device batch starts from and ends at (transcript.rs:226-243: state(),
 * counter(), fs_key()), with the running unmasked claim of the s(1) recovery. */
typedef struct {
    uint8_t state[32];
    uint64_t counter;
    uint8_t key[32];
    int32_t keyed;         /* 0: legacy unkeyed transcript */
    int32_t recover_one;   /* rounds.rs:81-86 */
    int32_t have_claim;    /* claim[] holds the exact unmasked sum for the first round of the batch */
    int32_t reserved;
    uint64_t claim[2];
} hl_fs_state;
/* `nd` consecutive rounds entirely on the device, as prove_rounds (rounds.rs:33-48) drives them under
 * a CfsMasker (sumcheck.rs:282-299): round sums, s(1) recovery, masked message s + c g_j, absorb
 * "sc-round", squeeze r_j, fold.  mask_coeffs NULL = no mask; otherwise mask_vars * degree + 2 Fp2 in
 * the layout of sumcheck.rs:199-200 and the batch must start at round 0.
 * out: per round (degree+1) unmasked sums, (degree+1) absorbed (masked) values, then r_j  (Fp2 each).
 * fs is updated to the position after the batch.  The caller replays the batch through its own
 * transcript and compares (metal.rs:4156-4171); nothing here is trusted blind. */
int hl_b200_rounds_batched(hl_rounds* r, uint32_t nd, hl_fs_state* fs, const uint64_t* mask_coeffs, uint32_t mask_vars,
                           const uint64_t mask_c[2], uint64_t* out);

/* ---- LogUp (hashline/src/private_block/protocol.rs:993-1011 inverses, :1928-1933 table_helper;
 * accuracy_act.rs:55-117 histogram / query_values / denominators) ----
 * Multiplicities: mult[v] = number of queries with idx == v, idx in [0, table_len). */
int hl_b200_logup_histogram(hl_ctx* ctx, const int32_t* idx, size_t nq, size_t table_len, uint64_t* mult);
/* Helper column h[i] = s_i / (alpha - ((idx_i + idx_off) + beta * out_i + tag)), an Fp2 per entry, with
 * s_i = 1 (mult NULL: the query side) or s_i = mult[i] (the table side m_v / (alpha - t_v); pass idx NULL
 * for idx_i = i).  Every term is formed in the field.  HL_B200_ERR_ZERO if ANY denominator is zero
 * ("zero LogUp denominator; discard attempt", protocol.rs:1005-1006); nothing is written then. */
int hl_b200_logup_helpers(hl_ctx* ctx, const int32_t* idx, const int32_t* outv, size_t n, const uint64_t alpha[2],
                          const uint64_t beta[2], const uint64_t tag[2], int64_t idx_off, const uint64_t* mult, uint64_t* h);

/* ---- the three-coordinate activation lookup of the accuracy lane (private_block/accuracy_act.rs:13-117) ----
 * Queries sit on rows of f_pad words (n = rows * f_pad); group(i) = group_ids[i % f_pad] when i / f_pad < tokens and
 * i % f_pad < hidden, else 0 (query_group, :52-54).  tables = groups x 4096 words (scaled_tables), groups 1 .. 4.
 * act_histogram (:61-79): counts[group * 4096 + gate + 2048]++ when the key is in range and tables[group][key] == output, else
 *   counts[0]++ and (*misses)++; every query counted, padding included.
 * act_helpers: h[i] = 1 / (alpha - (gate_i + 2048 + beta * output_i + beta^2 * group(i) + tag)) (denominators, :106-124, then
 *   protocol.rs:993 inverses); HL_B200_ERR_ZERO on a zero denominator, nothing written then.
 * act_table (:13-31 with protocol.rs:1928 table_helper): compressed[i] = (i % 4096) + beta * word_i + beta^2 * (i / 4096) + tag for
 *   i < groups * 4096, 2048 + tag up to len (a power of two); ht[i] = mult[i] / (alpha - compressed[i]).  compressed may be NULL. */
int hl_b200_act_histogram(hl_ctx* ctx, const int64_t* gates, const int64_t* outputs, size_t n, size_t f_pad, size_t tokens, size_t hidden,
                          const uint32_t* group_ids, const int64_t* tables, size_t groups, uint64_t* counts, uint64_t* misses);
int hl_b200_act_helpers(hl_ctx* ctx, const int64_t* gates, const int64_t* outputs, size_t n, size_t f_pad, size_t tokens, size_t hidden,
                        const uint32_t* group_ids, const uint64_t alpha[2], const uint64_t beta[2], const uint64_t tag[2], uint64_t* h);
int hl_b200_act_table(hl_ctx* ctx, const int64_t* tables, size_t groups, size_t len, const uint64_t* mult, const uint64_t alpha[2],
                      const uint64_t beta[2], const uint64_t tag[2], uint64_t* compressed, uint64_t* ht);

/* ---- witness weight products (hashline/src/gpu/metal.rs:4646-4680 witness_product; private_block/witness.rs:818-835 on_device,
 * :979-991 matmul_reference): out[t * os + j] = sum_i x[t * xs + i] * w(i, j) for t < t_rows, j < outer, with
 * w(i, j) = w[j * inner + i], or w[i * outer + j] when in_out; every other word of the out_len plane zero.  Exact: each
 * activation splits as 256 hi + lo (hi signed, lo unsigned byte), the two int8 products accumulate in int32 on the tensor
 * cores (|sum lo w| <= K * 32,640 < 2^31 for K <= 65,536, metal.rs:4234), and the plane is 256 P_hi + P_lo in int64.
 * *taken = 0 (and HL_B200_OK) when the CPU must take the product: an activation outside int16, or a shape outside
 * inner <= 65,536, xs >= inner, os >= outer, the rows inside x_len / out_len, inner * outer <= w_len.
 * The _dev form takes device pointers (weights resident in HBM across requests) and is asynchronous up to its own flag read. */
int hl_b200_witness_product(hl_ctx* ctx, size_t t_rows, const int64_t* x, size_t x_len, size_t xs, const int8_t* w, size_t w_len, size_t inner,
                            size_t outer, size_t os, size_t out_len, int in_out, int64_t* out, int* taken);
int hl_b200_witness_product_dev(hl_ctx* ctx, size_t t_rows, const int64_t* d_x, size_t x_len, size_t xs, const int8_t* d_w, size_t w_len, size_t inner,
                                size_t outer, size_t os, size_t out_len, int in_out, int64_t* d_out, int* taken);

/* ---- the masking commitment M of a block (hashline/src/zk.rs:447-536 mask_commit / mask_commit_tagged) and the product
 * polynomial of its opening (zk.rs:618-637 mask_open) ----
 * mask_commit: `msgs` = n_msg_rows rows of 2^log_msg EVALUATIONS (a mask's real or imaginary coefficients, its pads, zeros:
 * what zk.rs:466-470 assembles before `ntt.inverse`), `coef_rows` = n_coef_rows rows of 2^(log_msg + 1) COEFFICIENTS (b_re,
 * b_im, u_re, u_im with b[m] = -b[0] already set, zk.rs:478-483), `pows` = the 2^log_dom coset powers 7^i.  Every row is
 * evaluated on the coset (encode_coeffs_coset, zk.rs:441-445), columns are hashed under key32 (hash_columns[_keyed]).
 * Out: leaves32 (2^log_dom x 32 bytes, unsalted), a_coefs (n_msg_rows x 2^log_msg, the `a_coefs` of MaskCommit; may be
 * NULL) and a store whose data rows are the coefficient rows (2^(log_msg + 1) words each, message rows zero-extended):
 *   hl_b200_store_merkle            the salted tree (salt_leaf[_keyed], MerkleTree::build[_keyed])
 *   hl_b200_store_columns           the opened columns (zk.rs:650-654)
 *   hl_b200_store_fold(with_pads 0) the proximity combination (zk.rs:641-647) with weights (r_0 .. r_{rows-3}, 1, U)
 * log_msg 8 .. 11, log_dom - log_msg 1 .. 6; the reference's constants are 9 and 12.
 * mask_open_q: ws = n_masks x 2^log_msg Fp2 (combined_weights' vectors, zero-extended to the message length);
 * q = 2^(log_msg + 1) Fp2 = sum_s p_{a_s} p_{W_s} + p_b (zk.rs:623-637), rows 2s / 2s+1 the masks, rows 2 n_masks / +1 b. */
int hl_b200_mask_commit(hl_ctx* ctx, uint32_t log_msg, uint32_t log_dom, const uint64_t* msgs, size_t n_msg_rows, const uint64_t* coef_rows,
                        size_t n_coef_rows, const uint64_t* pows, const uint8_t* key32, hl_store** store, uint64_t* a_coefs, uint8_t* leaves32);
int hl_b200_mask_open_q(hl_store* store, size_t n_masks, const uint64_t* ws, uint64_t* q);

/* ---- LogUp helper columns of TABLE-INDEXED lookups (protocol.rs:1125-1230 u8_denominator_inverses, helper_one,
 * helper_pair_inverses_u8; :1700-1800 write_helpers_w16_cols): the byte tables and the range families ----
 * lookup_inverse_table: d_table[v] = 1 / (alpha - (v + g)) for v < 2^log_len (DEVICE memory, Fp2 per entry); an entry
 * whose denominator is zero is written as (0, 0) = absent, and does not refuse (protocol.rs:1122-1124).
 * lookup_helpers_dev: re[i], im[i] = the two words of entry_a(a[i]) (+ entry_b(b[i]) when d_b is given): the two planes
 * of H a helper job fills.  a, b: looked words as int64 in DEVICE memory; a word outside its table takes the direct
 * inversion (protocol.rs:1172-1180).  HL_B200_ERR_ZERO when a word's denominator is zero (its entry absent). */
int hl_b200_lookup_inverse_table(hl_ctx* ctx, const uint64_t alpha[2], const uint64_t g[2], uint32_t log_len, uint64_t* d_table);
int hl_b200_lookup_helpers_dev(hl_ctx* ctx, const int64_t* d_a, const uint64_t* d_table_a, uint32_t log_a, const uint64_t g_a[2],
                               const int64_t* d_b, const uint64_t* d_table_b, uint32_t log_b, const uint64_t g_b[2],
                               const uint64_t alpha[2], size_t n, uint64_t* d_re, uint64_t* d_im);

/* ---- weight folds (zkp-core/src/mle.rs:157-205 fold_rows_i8 / fold_cols_i8, deferred forms :256-319) ----
 * m: rows x cols int8, row-major.  fold_rows: out[j] = sum_i w[i] m[i][j] (w: rows Fp2, out: cols Fp2);
 * fold_cols: out[i] = sum_j c[j] m[i][j] (c: cols Fp2, out: rows Fp2).  Exact integer sums, one reduction. */
int hl_b200_fold_rows_i8(hl_ctx* ctx, const int8_t* m, size_t rows, size_t cols, const uint64_t* w, uint64_t* out);
int hl_b200_fold_cols_i8(hl_ctx* ctx, const int8_t* m, size_t rows, size_t cols, const uint64_t* c, uint64_t* out);

/* ---- counters: GpuStats / dev_stats (hashline/src/gpu/mod.rs:890-908) ---- */
typedef struct {
    uint64_t commits, folds, gathers, merkles, round_batches;
    uint64_t kernel_launches;   /* kernels this context has launched */
    uint64_t bytes_h2d, bytes_d2h;
    uint64_t declines;          /* calls that returned an error */
    uint64_t generated_rounds;  /* sumcheck rounds of slot programs that ran a generated per-graph kernel */
} hl_stats;
int hl_b200_stats(hl_ctx* ctx, hl_stats* out);

/* ---- per-kernel-family device time: the phase clock of timing.rs:1-130 / HL_METAL_TIMING
 * (metal.rs:2148-2179), taken with CUDA events on the context's stream.  Off by default. ---- */
enum { HL_T_ENCODE = 0, HL_T_HASH = 1, HL_T_MERKLE = 2, HL_T_FOLD = 3, HL_T_GATHER = 4, HL_T_ROUNDS = 5, HL_T_LOGUP = 6, HL_T_TABLES = 7, HL_T_WITNESS = 8, HL_T_COUNT = 9 };
typedef struct {
    double ms[HL_T_COUNT];        /* summed device time per family since the last reset */
    uint64_t spans[HL_T_COUNT];   /* timed spans per family (one span = the family's launches of one call) */
} hl_timing;
int hl_b200_timing_enable(hl_ctx* ctx, int on);
/* Waits for the stream, then reports (and with reset != 0 clears) the accumulated spans. */
int hl_b200_timing_read(hl_ctx* ctx, hl_timing* out, int reset);

#ifdef __cplusplus
}
#endif
#endif
