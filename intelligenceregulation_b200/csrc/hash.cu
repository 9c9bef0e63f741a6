// BLAKE3 kernels of the commitment: column leaves, salted leaves, Merkle levels.
//
// Column leaf j = BLAKE3[keyed](bytes of column j), the column's words taken row 0 first,
// eight little-endian bytes each (pcs.rs:176-221).  A 1 KiB BLAKE3 chunk is 128 rows of one
// column, a 64-byte block is 8 rows.  The matrix is row-major, so a warp that owns 32
// neighbouring columns reads 256 contiguous bytes per row: the column hash needs no transpose.
//
// Pass 1: one thread per (column, chunk) hashes its 128 rows into a chunk chaining value.
// Pass 2: one thread per column joins its chunk values along BLAKE3's tree (the left subtree
//         of a node is the largest power-of-two number of chunks below the node's size).
#include "b3.cuh"
#include "gl_field.cuh"
#include "kernels.h"

namespace {

__global__ void __launch_bounds__(128) k_hash_col_chunks(const u64* __restrict__ enc, u32 rows, u32 nn,
                                                         const uint32_t* __restrict__ key, u32 nchunks, u32 chunk0,
                                                         uint32_t* __restrict__ cvs, uint32_t* __restrict__ leaves) {
    const u32 col = blockIdx.x * blockDim.x + threadIdx.x, chunk = chunk0 + blockIdx.y;
    if (col >= nn) return;
    const u32 r0 = chunk * 128u, r1 = min(rows, r0 + 128u);
    const u32 nb = (r1 - r0 + 7u) / 8u;
    const uint32_t mode = key ? b3::KEYED : 0u;
    uint32_t cv[8];
    b3::init_cv(cv, key);
    const u64* p = enc + (size_t)r0 * nn + col;
    for (u32 b = 0; b < nb; b++) {
        uint32_t m[16];
        const u32 cnt = min(8u, r1 - r0 - 8u * b);
#pragma unroll
        for (u32 i = 0; i < 8; i++) {
            u64 w = i < cnt ? __ldcs(p + (size_t)(8u * b + i) * nn) : 0ull;
            m[2 * i] = (uint32_t)w;
            m[2 * i + 1] = (uint32_t)(w >> 32);
        }
        uint32_t flags = mode | (b == 0 ? b3::CHUNK_START : 0u);
        if (b == nb - 1) flags |= b3::CHUNK_END | (nchunks == 1 ? b3::ROOT : 0u);
        b3::compress(cv, m, chunk, cnt * 8u, flags);
    }
    uint32_t* dst = nchunks == 1 ? leaves + (size_t)col * 8 : cvs + ((size_t)chunk * nn + col) * 8;
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(cv[0], cv[1], cv[2], cv[3]);
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(cv[4], cv[5], cv[6], cv[7]);
}

__device__ __forceinline__ void parent(uint32_t (&out)[8], const uint32_t* l, const uint32_t* r, const uint32_t* key, bool root) {
    uint32_t m[16];
#pragma unroll
    for (int i = 0; i < 8; i++) { m[i] = l[i]; m[8 + i] = r[i]; }
    b3::init_cv(out, key);
    b3::compress(out, m, 0, 64, b3::PARENT | (key ? b3::KEYED : 0u) | (root ? b3::ROOT : 0u));
}

// Join nchunks (>= 2) chunk values per column.  Complete power-of-two subtrees are joined as
// soon as both halves exist (a binary counter over the chunks seen); what remains at the end
// is joined from the right, and the last join carries the ROOT flag.
__global__ void __launch_bounds__(128) k_hash_col_merge(const uint32_t* __restrict__ cvs, u32 nn, u32 nchunks,
                                                        const uint32_t* __restrict__ key, uint32_t* __restrict__ leaves) {
    const u32 col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= nn) return;
    uint32_t stack[24][8];
    int sp = 0;
    for (u32 c = 0; c < nchunks; c++) {
        const uint4* src = reinterpret_cast<const uint4*>(cvs + ((size_t)c * nn + col) * 8);
        uint4 a = src[0], b = src[1];
        uint32_t* top = stack[sp++];
        top[0] = a.x; top[1] = a.y; top[2] = a.z; top[3] = a.w;
        top[4] = b.x; top[5] = b.y; top[6] = b.z; top[7] = b.w;
        if (c + 1 == nchunks) break;
        for (u32 t = c + 1; (t & 1u) == 0; t >>= 1) {  // one join per trailing zero of the count
            uint32_t out[8];
            parent(out, stack[sp - 2], stack[sp - 1], key, false);
            sp--;
#pragma unroll
            for (int i = 0; i < 8; i++) stack[sp - 1][i] = out[i];
        }
    }
    while (sp > 1) {
        uint32_t out[8];
        parent(out, stack[sp - 2], stack[sp - 1], key, sp == 2);
        sp--;
#pragma unroll
        for (int i = 0; i < 8; i++) stack[sp - 1][i] = out[i];
    }
    uint32_t* dst = leaves + (size_t)col * 8;
#pragma unroll
    for (int i = 0; i < 8; i++) dst[i] = stack[0][i];
}

// dst[j] = H_key(a[j] || b[j]) for 32-byte a, b: salted leaves (a = leaves, b = salts) and
// tree levels (a = even nodes, b = odd nodes of the level below); pcs.rs:696-715, merkle.rs:14-31
__global__ void k_hash_pairs(const uint32_t* __restrict__ a, const uint32_t* __restrict__ b, size_t stride_words,
                             u32 count, const uint32_t* __restrict__ key, uint32_t* __restrict__ dst) {
    const u32 j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= count) return;
    uint32_t m[16], out[8];
    const uint4* pa = reinterpret_cast<const uint4*>(a + (size_t)j * stride_words);
    const uint4* pb = reinterpret_cast<const uint4*>(b + (size_t)j * stride_words);
    uint4 x = pa[0], y = pa[1], z = pb[0], w = pb[1];
    m[0] = x.x; m[1] = x.y; m[2] = x.z; m[3] = x.w; m[4] = y.x; m[5] = y.y; m[6] = y.z; m[7] = y.w;
    m[8] = z.x; m[9] = z.y; m[10] = z.z; m[11] = z.w; m[12] = w.x; m[13] = w.y; m[14] = w.z; m[15] = w.w;
    b3::hash64(out, m, key);
    uint4* pd = reinterpret_cast<uint4*>(dst + (size_t)j * 8);
    pd[0] = make_uint4(out[0], out[1], out[2], out[3]);
    pd[1] = make_uint4(out[4], out[5], out[6], out[7]);
}

// The top of the tree in one CTA: from a level of `width` (<= 2048) nodes down to the root.
__global__ void __launch_bounds__(1024) k_merkle_top(uint32_t* __restrict__ levels, size_t level_off_words, u32 width,
                                                     const uint32_t* __restrict__ key) {
    size_t off = level_off_words;
    for (u32 w = width; w > 1; w >>= 1) {
        const uint32_t* src = levels + off;
        uint32_t* dst = levels + off + (size_t)w * 8;
        for (u32 j = threadIdx.x; j < w / 2; j += blockDim.x) {
            uint32_t m[16], out[8];
#pragma unroll
            for (int i = 0; i < 16; i++) m[i] = src[(size_t)j * 16 + i];
            b3::hash64(out, m, key);
#pragma unroll
            for (int i = 0; i < 8; i++) dst[(size_t)j * 8 + i] = out[i];
        }
        off += (size_t)w * 8;
        __syncthreads();
    }
}

// Salted leaves and the lowest levels of the tree in one launch: a CTA owns SUB consecutive leaves, salts them (or takes them as
// they are when there are no salts), and hashes its subtree level by level through shared memory, writing every level to its place
// in `levels`; k_merkle_top then joins the nn / SUB subtree roots.  Two launches for a tree instead of one per level.
constexpr u32 SUBTREE = 512, SUBTREE_T = 256;
__global__ void __launch_bounds__(SUBTREE_T) k_merkle_subtrees(const uint32_t* __restrict__ leaves, const uint32_t* __restrict__ salts, u32 nn,
                                                               const uint32_t* __restrict__ leaf_key, const uint32_t* __restrict__ node_key,
                                                               uint32_t* __restrict__ levels) {
    __shared__ uint4 buf[2][SUBTREE][2];  // two levels of 32-byte nodes
    const u32 first = blockIdx.x * SUBTREE;
    for (u32 t = threadIdx.x; t < SUBTREE; t += SUBTREE_T) {
        const uint4* pl = reinterpret_cast<const uint4*>(leaves + (size_t)(first + t) * 8);
        uint4 a = pl[0], b = pl[1];
        if (salts) {
            const uint4* ps = reinterpret_cast<const uint4*>(salts + (size_t)(first + t) * 8);
            const uint4 z = ps[0], w = ps[1];
            uint32_t m[16] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w, z.x, z.y, z.z, z.w, w.x, w.y, w.z, w.w}, out[8];
            b3::hash64(out, m, leaf_key);
            a = make_uint4(out[0], out[1], out[2], out[3]);
            b = make_uint4(out[4], out[5], out[6], out[7]);
        }
        buf[0][t][0] = a; buf[0][t][1] = b;
        uint4* pd = reinterpret_cast<uint4*>(levels + (size_t)(first + t) * 8);
        pd[0] = a; pd[1] = b;
    }
    __syncthreads();
    size_t off = (size_t)nn * 8;  // words before the level being written
    u32 cur = 0, level_w = nn >> 1;
    for (u32 w = SUBTREE >> 1; w >= 1; w >>= 1) {
        for (u32 j = threadIdx.x; j < w; j += SUBTREE_T) {
            const uint4 x = buf[cur][2 * j][0], y = buf[cur][2 * j][1], z = buf[cur][2 * j + 1][0], v = buf[cur][2 * j + 1][1];
            uint32_t m[16] = {x.x, x.y, x.z, x.w, y.x, y.y, y.z, y.w, z.x, z.y, z.z, z.w, v.x, v.y, v.z, v.w}, out[8];
            b3::hash64(out, m, node_key);
            const uint4 a = make_uint4(out[0], out[1], out[2], out[3]), b = make_uint4(out[4], out[5], out[6], out[7]);
            buf[cur ^ 1][j][0] = a; buf[cur ^ 1][j][1] = b;
            uint4* pd = reinterpret_cast<uint4*>(levels + off + ((size_t)blockIdx.x * w + j) * 8);
            pd[0] = a; pd[1] = b;
        }
        __syncthreads();
        off += (size_t)level_w * 8;
        level_w >>= 1;
        cur ^= 1;
    }
}

}  // namespace

namespace hlk {

// salted leaves (salts may be NULL: the leaves are the lowest level as they are) and every level above them
cudaError_t merkle_tree(const uint32_t* d_leaves, const uint32_t* d_salts, u32 nn, const uint32_t* d_leaf_key, const uint32_t* d_node_key,
                        uint32_t* d_levels, cudaStream_t st, int* launches) {
    if (nn >= 2 * SUBTREE && nn / SUBTREE <= 2048) {
        k_merkle_subtrees<<<nn / SUBTREE, SUBTREE_T, 0, st>>>(d_leaves, d_salts, nn, d_leaf_key, d_node_key, d_levels);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        size_t off = 0;  // words before the level of the subtree roots
        for (u32 w = nn; w > nn / SUBTREE; w >>= 1) off += (size_t)w * 8;
        k_merkle_top<<<1, 1024, 0, st>>>(d_levels, off, nn / SUBTREE, d_node_key);
        *launches = 2;
        return cudaGetLastError();
    }
    cudaError_t e = d_salts ? salt_leaves(d_leaves, d_salts, nn, d_leaf_key, d_levels, st)
                            : cudaMemcpyAsync(d_levels, d_leaves, (size_t)nn * 32, cudaMemcpyDeviceToDevice, st);
    *launches = d_salts ? 1 : 0;
    if (e != cudaSuccess) return e;
    for (u32 w = nn; w > 2048; w >>= 1) (*launches)++;
    if (nn > 1) (*launches)++;
    return merkle_levels(d_levels, nn, d_node_key, st);
}

u32 hash_chunks(u32 rows) { return (rows + 127u) / 128u; }

cudaError_t hash_columns(const u64* enc, u32 rows, u32 nn, const uint32_t* d_key, uint32_t* d_cvs, uint32_t* d_leaves,
                         cudaStream_t st) {
    const u32 nchunks = hash_chunks(rows);
    cudaError_t e = hash_column_chunks(enc, rows, nn, d_key, 0, nchunks, d_cvs, d_leaves, st);
    if (e != cudaSuccess || nchunks == 1) return e;
    return hash_column_merge(rows, nn, d_key, d_cvs, d_leaves, st);
}

// the chunk values of the 1 KiB chunks [chunk0, chunk0 + count) of every column (rows 128 chunk0 .. of the encoding
// must be complete); a commitment whose rows arrive in pieces hashes each piece as soon as it is encoded
cudaError_t hash_column_chunks(const u64* enc, u32 rows, u32 nn, const uint32_t* d_key, u32 chunk0, u32 count, uint32_t* d_cvs,
                               uint32_t* d_leaves, cudaStream_t st) {
    if (count == 0) return cudaSuccess;
    dim3 grid((nn + 127u) / 128u, count);
    k_hash_col_chunks<<<grid, 128, 0, st>>>(enc, rows, nn, d_key, hash_chunks(rows), chunk0, d_cvs, d_leaves);
    return cudaGetLastError();
}

cudaError_t hash_column_merge(u32 rows, u32 nn, const uint32_t* d_key, const uint32_t* d_cvs, uint32_t* d_leaves, cudaStream_t st) {
    k_hash_col_merge<<<(nn + 127u) / 128u, 128, 0, st>>>(d_cvs, nn, hash_chunks(rows), d_key, d_leaves);
    return cudaGetLastError();
}

// levels: (2 nn - 1) x 8 words; level 0 (nn salted leaves) must already be in place
cudaError_t merkle_levels(uint32_t* d_levels, u32 nn, const uint32_t* d_node_key, cudaStream_t st) {
    size_t off = 0;
    u32 w = nn;
    while (w > 2048) {
        const uint32_t* src = d_levels + off;
        uint32_t* dst = d_levels + off + (size_t)w * 8;
        k_hash_pairs<<<(w / 2 + 127u) / 128u, 128, 0, st>>>(src, src + 8, 16, w / 2, d_node_key, dst);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        off += (size_t)w * 8;
        w >>= 1;
    }
    if (w > 1) {
        k_merkle_top<<<1, 1024, 0, st>>>(d_levels, off, w, d_node_key);
        return cudaGetLastError();
    }
    return cudaSuccess;
}

cudaError_t salt_leaves(const uint32_t* d_leaves, const uint32_t* d_salts, u32 nn, const uint32_t* d_leaf_key,
                        uint32_t* d_out, cudaStream_t st) {
    k_hash_pairs<<<(nn + 127u) / 128u, 128, 0, st>>>(d_leaves, d_salts, 8, nn, d_leaf_key, d_out);
    return cudaGetLastError();
}

}  // namespace hlk
