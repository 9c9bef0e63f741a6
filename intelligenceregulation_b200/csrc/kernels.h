// Launch wrappers of the device kernels (one .cu file per family).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "encode_core.cuh"

namespace hlk {

// encode.cu
size_t encode_scratch_words(u32 logn, u32 T, int sm_count, u32 rows);
cudaError_t encode_rows(const enc::RowArgs& a, u32 logn, bool allow_fast, int sm_count, size_t scratch_words,
                        cudaStream_t st, int* path_out);
cudaError_t widen_rows(const unsigned char* narrow, const u64* row_off, const unsigned char* row_w, u64* out, u32 rows, u32 n, int sm_count, cudaStream_t st);
cudaError_t encode_rows_form(const enc::RowArgs& a, u32 logn, int form, int sm_count, size_t scratch_words, cudaStream_t st);

// hash.cu
u32 hash_chunks(u32 rows);
cudaError_t hash_column_chunks(const u64* enc, u32 rows, u32 nn, const uint32_t* d_key, u32 chunk0, u32 count, uint32_t* d_cvs,
                               uint32_t* d_leaves, cudaStream_t st);
cudaError_t hash_column_merge(u32 rows, u32 nn, const uint32_t* d_key, const uint32_t* d_cvs, uint32_t* d_leaves, cudaStream_t st);
cudaError_t hash_columns(const u64* enc, u32 rows, u32 nn, const uint32_t* d_key, uint32_t* d_cvs, uint32_t* d_leaves,
                         cudaStream_t st);
cudaError_t salt_leaves(const uint32_t* d_leaves, const uint32_t* d_salts, u32 nn, const uint32_t* d_leaf_key,
                        uint32_t* d_out, cudaStream_t st);
cudaError_t merkle_levels(uint32_t* d_levels, u32 nn, const uint32_t* d_node_key, cudaStream_t st);
cudaError_t merkle_tree(const uint32_t* d_leaves, const uint32_t* d_salts, u32 nn, const uint32_t* d_leaf_key, const uint32_t* d_node_key,
                        uint32_t* d_levels, cudaStream_t st, int* launches);

// store.cu
// out[g] = rho_g^T [src | src2]: ncols entries from src (element (i, j) at src[i ld + j ir]), then ncols2 from src2 (may be NULL)
// rows cut into `splits` ranges (fold_row_splits: > 1 when a few dense vectors would leave the machine short of loads in flight);
// d_part = splits x k x out_ld Fp2 of scratch when splits > 1
u32 fold_row_splits(u32 rows, u32 ncols, u32 ncols2, u32 k, int sm_count);
// one or two dense vectors over contiguous rows in one memory-shaped pass: fold_few_ranges > 0 when it applies (d_part = ranges x k x
// out_ld Fp2 of scratch)
u32 fold_few_ranges(u32 rows, u32 ncols, u32 ncols2, u32 k, u32 ir, int sm_count);
cudaError_t fold_rows_few(const u64* src, u32 rows, u32 ncols, size_t ld, const u64* src2, u32 ncols2, size_t ld2, const u64* d_rhos, u32 k,
                          const u32* d_out_map, u64* d_out, u32 out_ld, u32 ranges, u64* d_part, cudaStream_t st);
cudaError_t fold_rows(const u64* src, u32 rows, u32 ncols, size_t ld, u32 ir, const u64* src2, u32 ncols2, size_t ld2, const u64* d_rhos, u32 k,
                      const u32* d_out_map, u64* d_out, u32 out_ld, cudaStream_t st, u32 splits = 1, u64* d_part = nullptr);
cudaError_t fold_rows_sparse(const u64* src, u32 ncols, size_t ld, u32 ir, const u64* src2, u32 ncols2, size_t ld2, const u32* d_off,
                             const u32* d_rows, const u64* d_weights, u32 k, const u32* d_out_map, u64* d_out, u32 out_ld, cudaStream_t st);
cudaError_t gather_columns(const u64* enc, u32 rows, size_t nn, const u64* d_idx, u32 nidx, u64* d_out, cudaStream_t st);

// misc.cu
cudaError_t probe_field(const u64* d_a, const u64* d_b, size_t n, u64* d_out3, cudaStream_t st);
cudaError_t butterfly_peak(const u64* d_seed, u64* d_sink, u32 iters, int blocks, cudaStream_t st);
cudaError_t compress_peak(const u64* d_seed, u64* d_sink, u32 iters, int blocks, cudaStream_t st);

}  // namespace hlk
