// The verifier's per-column checks of a hiding opening on the device (pcs.rs:1303-1331, `verify_zk_tagged`'s parallel map
// over the opened columns).  For each opened column (j, col, salt, path) the reference computes
//     leaf = H_leaf(H_column(col) || salt),  walks `path` from position j to the root (merkle.rs:120-127),
//     and for every combined row weight rho_g checks  rho_g^T col == encode(clear vector g)[j]  (a26_combine, pcs.rs:1322-1328).
// The checks that come before the map (path lengths, vector lengths, <v, c> against the claims, the Fiat-Shamir draws of rho
// and of the indices) are transcript work and stay with the caller.
//
// Layout: the caller's columns are ncols runs of `rows` words.  They are transposed once into a rows x ncols matrix, which is
// the layout the commitment's own column hash and row fold read (32 neighbouring columns per warp and row), so the two heavy
// parts run through the same kernels as the prover's.  One thread per column then salts the leaf, walks the path and compares
// the combinations; it writes one verdict word per column.
#include <vector>

#include "api_internal.h"
#include "b3.cuh"
#include "gl_field.cuh"

using namespace hlapi;

namespace {

// in: ncols x rows, out: rows x ncols
__global__ void __launch_bounds__(256) k_cols_to_rows(const u64* __restrict__ in, u32 ncols, u32 rows, u64* __restrict__ out) {
    __shared__ u64 tile[32][33];
    const u32 r0 = blockIdx.x * 32u, c0 = blockIdx.y * 32u;
    for (u32 y = threadIdx.y; y < 32u; y += 8u) {
        const u32 c = c0 + y, r = r0 + threadIdx.x;
        tile[y][threadIdx.x] = (c < ncols && r < rows) ? in[(size_t)c * rows + r] : 0ull;
    }
    __syncthreads();
    for (u32 y = threadIdx.y; y < 32u; y += 8u) {
        const u32 r = r0 + y, c = c0 + threadIdx.x;
        if (r < rows && c < ncols) out[(size_t)r * ncols + c] = tile[threadIdx.x][y];
    }
}

// verdict[c]: 0 all checks hold; 1 the Merkle path fails; 2 + g the column disagrees with clear vector g (the first such g).
// The order is the reference's: the path is checked before the combinations.
// wants: k x ncols Fp2 from the caller, or (wants == NULL) rows 2g / 2g + 1 of `enc` (row length nn) at position idx[c].
__global__ void __launch_bounds__(128) k_verify_columns(const uint32_t* __restrict__ leaves, const uint32_t* __restrict__ salts,
                                                        const uint32_t* __restrict__ paths, u32 depth, const u64* __restrict__ idx,
                                                        const uint32_t* __restrict__ root, const uint32_t* __restrict__ leaf_key,
                                                        const uint32_t* __restrict__ node_key, const u64* __restrict__ acc, u32 k,
                                                        const u64* __restrict__ wants, const u64* __restrict__ enc, size_t nn, u32 ncols,
                                                        int32_t* __restrict__ verdict) {
    const u32 c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= ncols) return;
    uint32_t m[16], cur[8];
#pragma unroll
    for (int i = 0; i < 8; i++) { m[i] = leaves[(size_t)c * 8 + i]; m[8 + i] = salts[(size_t)c * 8 + i]; }
    b3::hash64(cur, m, leaf_key);
    u64 pos = idx[c];
    for (u32 l = 0; l < depth; l++) {
        const uint32_t* sib = paths + ((size_t)c * depth + l) * 8;
        const bool right = pos & 1ull;  // this node is the right child: the sibling goes first
#pragma unroll
        for (int i = 0; i < 8; i++) { m[i] = right ? sib[i] : cur[i]; m[8 + i] = right ? cur[i] : sib[i]; }
        b3::hash64(cur, m, node_key);
        pos >>= 1;
    }
    bool ok = true;
#pragma unroll
    for (int i = 0; i < 8; i++) ok = ok && cur[i] == root[i];
    int32_t v = ok ? 0 : 1;
    if (ok) {
        const u64 j = idx[c];
        for (u32 g = 0; g < k; g++) {
            const u64 a0 = acc[((size_t)g * ncols + c) * 2], a1 = acc[((size_t)g * ncols + c) * 2 + 1];
            u64 w0, w1;
            if (wants) { w0 = wants[((size_t)g * ncols + c) * 2]; w1 = wants[((size_t)g * ncols + c) * 2 + 1]; }
            else { w0 = enc[(size_t)(2 * g) * nn + j]; w1 = enc[(size_t)(2 * g + 1) * nn + j]; }
            if (a0 != w0 || a1 != w1) { v = 2 + (int32_t)g; break; }
        }
    }
    verdict[c] = v;
}

// vecs: k vectors of n + q Fp2 -> 2k base rows (re of vector 0, im of vector 0, re of vector 1, ..): the first n words of each into
// `data` (2k x n), the last q into `pads` (2k x q), the rows a hiding commitment takes (pcs.rs:1287-1296)
__global__ void __launch_bounds__(256) k_split_vectors(const u64* __restrict__ vecs, u32 k, u32 n, u32 q, u64* __restrict__ data, u64* __restrict__ pads) {
    const u32 g = blockIdx.y, w = n + q;
    for (u32 j = blockIdx.x * blockDim.x + threadIdx.x; j < w; j += gridDim.x * blockDim.x) {
        const u64 re = vecs[((size_t)g * w + j) * 2], im = vecs[((size_t)g * w + j) * 2 + 1];
        if (j < n) {
            data[(size_t)(2 * g) * n + j] = re;
            data[(size_t)(2 * g + 1) * n + j] = im;
        } else {
            pads[(size_t)(2 * g) * q + (j - n)] = re;
            pads[(size_t)(2 * g + 1) * q + (j - n)] = im;
        }
    }
    (void)k;
}

}  // namespace

// the body of hl_b200_verify_columns; the caller holds the context's lock
static int verify_columns_locked(hl_ctx* c, const uint64_t* cols, size_t rows, size_t ncols, const uint64_t* idx, const uint8_t* salts32,
                                 const uint8_t* paths32, uint32_t depth, const uint8_t* root32, const uint8_t* column_key32,
                                 const uint8_t* leaf_key32, const uint8_t* node_key32, const uint64_t* rhos, size_t k, const uint64_t* wants,
                                 const hl_store* vec_store, int32_t* verdict, int64_t* first_bad) {
    if (!cols || !idx || !salts32 || !root32 || !verdict || rows == 0 || ncols == 0) return fail(c, HL_B200_ERR_ARG, "verify_columns: null or empty argument");
    if (depth && !paths32) return fail(c, HL_B200_ERR_ARG, "verify_columns: paths missing");
    if (depth > 40) return fail(c, HL_B200_ERR_ARG, "verify_columns: a path of more than 40 entries");
    if (k && !rhos) return fail(c, HL_B200_ERR_ARG, "verify_columns: row weights missing");
    if (k && ((wants != nullptr) == (vec_store != nullptr))) return fail(c, HL_B200_ERR_ARG, "verify_columns: give the expected values or the vectors' store, one of the two");
    if (rows > 0x7FFFFFFFu || ncols > 0x7FFFFFFFu || k > 0xFFFFu * 8u) return fail(c, HL_B200_ERR_ARG, "verify_columns: size");
    if (k && vec_store) {
        if (vec_store->ctx != c) return fail(c, HL_B200_ERR_ARG, "verify_columns: the vectors' store belongs to another context");
        if (vec_store->rows < 2 * k) return fail(c, HL_B200_ERR_ARG, "verify_columns: the vectors' store has fewer than 2k rows");
        // an index beyond the encoding is the caller's "column index != sampled" case; it must not become a device read
        for (size_t i = 0; i < ncols; i++)
            if (idx[i] >= vec_store->nn()) return fail(c, HL_B200_ERR_ARG, "verify_columns: a column index beyond the encoding");
    }
    const size_t cb = rows * ncols * 8, pb = (size_t)(depth ? depth : 1) * ncols * 32, ab = (k ? k : 1) * ncols * 16;
    const u32 nchunks = hlk::hash_chunks((u32)rows);
    const size_t cvs_bytes = nchunks > 1 ? (size_t)nchunks * ncols * 32 : 0;
    u64 *d_cols = nullptr, *d_mat = nullptr, *d_idx = nullptr, *d_rhos = nullptr, *d_acc = nullptr, *d_wants = nullptr;
    uint32_t *d_salts = nullptr, *d_paths = nullptr, *d_root = nullptr, *d_ck = nullptr, *d_lk = nullptr, *d_nk = nullptr, *d_leaves = nullptr, *d_cvs = nullptr;
    int32_t* d_verdict = nullptr;
    int rc = dev_alloc(c, (void**)&d_cols, cb);
    if (!rc) rc = dev_alloc(c, (void**)&d_mat, cb);
    if (!rc) rc = dev_alloc(c, (void**)&d_idx, ncols * 8);
    if (!rc) rc = dev_alloc(c, (void**)&d_salts, ncols * 32);
    if (!rc) rc = dev_alloc(c, (void**)&d_paths, pb);
    if (!rc) rc = dev_alloc(c, (void**)&d_root, 32);
    if (!rc) rc = dev_alloc(c, (void**)&d_leaves, ncols * 32);
    if (!rc && cvs_bytes) rc = dev_alloc(c, (void**)&d_cvs, cvs_bytes);
    if (!rc) rc = dev_alloc(c, (void**)&d_acc, ab);
    if (!rc) rc = dev_alloc(c, (void**)&d_verdict, ncols * 4);
    if (!rc && k) rc = dev_alloc(c, (void**)&d_rhos, k * rows * 16);
    if (!rc && k && wants) rc = dev_alloc(c, (void**)&d_wants, ab);
    if (!rc) rc = h2d(c, d_cols, cols, cb);
    if (!rc) rc = h2d(c, d_idx, idx, ncols * 8);
    if (!rc) rc = h2d(c, d_salts, salts32, ncols * 32);
    if (!rc && depth) rc = h2d(c, d_paths, paths32, (size_t)depth * ncols * 32);
    if (!rc) rc = h2d(c, d_root, root32, 32);
    if (!rc && k) rc = h2d(c, d_rhos, rhos, k * rows * 16);
    if (!rc && d_wants) rc = h2d(c, d_wants, wants, ab);
    if (!rc) rc = upload_key(c, column_key32, &d_ck);
    if (!rc) rc = upload_key(c, leaf_key32, &d_lk);
    if (!rc) rc = upload_key(c, node_key32, &d_nk);
    if (!rc) {
        const dim3 grid((unsigned)((rows + 31) / 32), (unsigned)((ncols + 31) / 32));
        k_cols_to_rows<<<grid, dim3(32, 8), 0, c->stream>>>(d_cols, (u32)ncols, (u32)rows, d_mat);
        cudaError_t e = cudaGetLastError();
        if (e == cudaSuccess) {
            Timed t(c, HL_T_HASH);
            e = hlk::hash_columns(d_mat, (u32)rows, (u32)ncols, d_ck, d_cvs, d_leaves, c->stream);
        }
        if (e == cudaSuccess && k) {
            Timed t(c, HL_T_FOLD);
            e = hlk::fold_rows(d_mat, (u32)rows, (u32)ncols, ncols, 1u, nullptr, 0u, 0, d_rhos, (u32)k, nullptr, d_acc, (u32)ncols, c->stream);
        }
        if (e == cudaSuccess) {
            k_verify_columns<<<(unsigned)((ncols + 127) / 128), 128, 0, c->stream>>>(
                d_leaves, d_salts, d_paths, depth, d_idx, d_root, d_lk, d_nk, d_acc, (u32)k, d_wants, vec_store ? vec_store->d_enc : nullptr,
                vec_store ? vec_store->nn() : 0, (u32)ncols, d_verdict);
            e = cudaGetLastError();
        }
        c->stats.kernel_launches += 2 + (nchunks > 1 ? 2 : 1) + (k ? 1 : 0);
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "verify_columns launch", e);
    }
    if (!rc) rc = d2h(c, verdict, d_verdict, ncols * 4);
    if (!rc) rc = sync(c, "verify_columns");
    if (!rc && first_bad) {
        *first_bad = -1;
        for (size_t i = 0; i < ncols; i++)
            if (verdict[i]) { *first_bad = (int64_t)i; break; }
    }
    if (rc) cudaStreamSynchronize(c->stream);  // copies already queued read the caller's memory: none outlives the call
    dev_free(c, d_cols, cb); dev_free(c, d_mat, cb); dev_free(c, d_idx, ncols * 8); dev_free(c, d_salts, ncols * 32);
    dev_free(c, d_paths, pb); dev_free(c, d_root, 32); dev_free(c, d_leaves, ncols * 32);
    if (d_cvs) dev_free(c, d_cvs, cvs_bytes);
    dev_free(c, d_acc, ab); dev_free(c, d_verdict, ncols * 4);
    if (d_rhos) dev_free(c, d_rhos, k * rows * 16);
    if (d_wants) dev_free(c, d_wants, ab);
    if (d_ck) dev_free(c, d_ck, 32);
    if (d_lk) dev_free(c, d_lk, 32);
    if (d_nk) dev_free(c, d_nk, 32);
    return rc;
}

extern "C" int hl_b200_verify_columns(hl_ctx* c, const uint64_t* cols, size_t rows, size_t ncols, const uint64_t* idx, const uint8_t* salts32,
                                      const uint8_t* paths32, uint32_t depth, const uint8_t* root32, const uint8_t* column_key32,
                                      const uint8_t* leaf_key32, const uint8_t* node_key32, const uint64_t* rhos, size_t k, const uint64_t* wants,
                                      const hl_store* vec_store, int32_t* verdict, int64_t* first_bad) {
    if (!c) return HL_B200_ERR_ARG;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    return verify_columns_locked(c, cols, rows, ncols, idx, salts32, paths32, depth, root32, column_key32, leaf_key32, node_key32, rhos, k, wants, vec_store,
                                 verdict, first_bad);
}

extern "C" int hl_b200_verify_opening(hl_ctx* c, uint32_t log_cols, uint32_t inv_rate, size_t q, const uint64_t* pows, const uint64_t* vecs, size_t k,
                                      const uint64_t* cols, size_t rows, size_t ncols, const uint64_t* idx, const uint8_t* salts32,
                                      const uint8_t* paths32, uint32_t depth, const uint8_t* root32, const uint8_t* column_key32,
                                      const uint8_t* leaf_key32, const uint8_t* node_key32, const uint64_t* rhos, int32_t* verdict, int64_t* first_bad) {
    if (!c) return HL_B200_ERR_ARG;
    if (!pows || !vecs || k == 0 || q == 0) return fail(c, HL_B200_ERR_ARG, "verify_opening: null or empty argument");
    if (log_cols < 1 || log_cols > 16 || k > 0x7FFFu) return fail(c, HL_B200_ERR_ARG, "verify_opening: shape");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    const size_t n = (size_t)1 << log_cols, nn = n * inv_rate, w = n + q;
    u64 *d_vecs = nullptr, *d_data = nullptr, *d_pads = nullptr, *d_pows = nullptr;
    hl_store* st = nullptr;
    int rc = dev_alloc(c, (void**)&d_vecs, k * w * 16);
    if (!rc) rc = dev_alloc(c, (void**)&d_data, 2 * k * n * 8);
    if (!rc) rc = dev_alloc(c, (void**)&d_pads, 2 * k * q * 8);
    if (!rc) rc = dev_alloc(c, (void**)&d_pows, nn * 8);
    if (!rc) rc = h2d(c, d_vecs, vecs, k * w * 16);
    if (!rc) rc = h2d(c, d_pows, pows, nn * 8);
    if (!rc) {
        const unsigned bx = (unsigned)((w + 255) / 256 < 64 ? (w + 255) / 256 : 64);
        k_split_vectors<<<dim3(bx, (unsigned)k), 256, 0, c->stream>>>(d_vecs, (u32)k, (u32)n, (u32)q, d_data, d_pads);
        c->stats.kernel_launches++;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "verify_opening launch", e);
    }
    // the commitment's own encoder on the 2k rows; the shape checks (inv_rate a power of two, n + q <= nn) are its
    if (!rc) rc = commit_resident(c, log_cols, inv_rate, d_data, 2 * k, d_pads, q, d_pows, nullptr, &st, nullptr);
    if (!rc)
        rc = verify_columns_locked(c, cols, rows, ncols, idx, salts32, paths32, depth, root32, column_key32, leaf_key32, node_key32, rhos, k, nullptr, st,
                                   verdict, first_bad);
    if (rc) cudaStreamSynchronize(c->stream);  // a refusal on the way: the copies above may still be reading the caller's memory
    if (st) store_release(st);
    dev_free(c, d_vecs, k * w * 16);
    dev_free(c, d_data, 2 * k * n * 8);
    dev_free(c, d_pads, 2 * k * q * 8);
    dev_free(c, d_pows, nn * 8);
    return rc;
}
