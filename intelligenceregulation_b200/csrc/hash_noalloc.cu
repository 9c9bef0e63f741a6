// hl_b200_hash_columns_static: the BLAKE3 column-leaf hash for callers that must not allocate.
//
// Who needs it: a prover thread that is handed device buffers by someone else and runs where device
// allocation is off limits - inside a latency-critical serving loop whose memory was carved out up front,
// under a host allocator cap that is already spent, or in a plug-in whose embedding process owns the CUDA
// memory pools.  For those callers a hidden cudaMalloc (even a pooled, stream-ordered one) is either
// forbidden or an unpredictable stall.  The regular path (hl_b200_commit*) allocates the per-chunk
// chaining-value scratch on every call; this variant keeps that scratch in a fixed array that lives in the
// library image instead, so the call itself allocates nothing: no cudaMalloc / cudaFree, no memory pool,
// no allocating library routine.  The caller passes the encoded matrix and the output leaves, both already
// on the device.
//
// Cost and limits: the array below occupies HL_B200_STATIC_CV_BYTES (24 MiB) on every GPU that loads this
// library, from load until the process exits.  A call needs ceil(rows / 128) * nn chaining values of 32
// bytes; larger shapes are refused with HL_B200_ERR_UNSUPPORTED (the Llama-3-8B block shape, 20 chunks x
// 32,768 columns = 20 MiB, fits).  All calls on a device share the one array and it keeps whatever the last
// call left there.  Nothing in it has to start at zero: pass 1 writes every value pass 2 reads.  Two calls
// whose kernels overlap on the same GPU (different streams, or different host threads) race on it and
// produce garbage leaves; serialise them.
//
// Set-up: host code cannot use the array's name as a device address (on the host it is only a stand-in
// symbol; a kernel handed it would fault or scribble over unrelated memory), so the first call on each
// device asks the runtime for the real address with cudaGetSymbolAddress, with that device current, and
// caches it.  That first call should therefore happen before any stream capture begins.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/hl_b200.h"
#include "b3.cuh"
#include "gl_field.cuh"

#define HL_B200_STATIC_CV_BYTES (24u << 20)

static __device__ __align__(256) unsigned char g_static_cv[HL_B200_STATIC_CV_BYTES];

namespace {

struct Key8 {
    uint32_t w[8];
    int keyed;
};

// pass 1: one thread per (column, 1 KiB chunk = 128 rows); same hashing rule as the allocating path
__global__ void __launch_bounds__(128) k_static_col_chunks(const u64* __restrict__ enc, u32 rows, u32 nn, Key8 key, u32 nchunks,
                                                           uint32_t* __restrict__ cvs, uint32_t* __restrict__ leaves) {
    const u32 col = blockIdx.x * blockDim.x + threadIdx.x, chunk = blockIdx.y;
    if (col >= nn) return;
    const u32 r0 = chunk * 128u, r1 = min(rows, r0 + 128u), nb = (r1 - r0 + 7u) / 8u;
    const uint32_t mode = key.keyed ? b3::KEYED : 0u;
    uint32_t cv[8];
#pragma unroll
    for (int i = 0; i < 8; i++) cv[i] = key.keyed ? key.w[i] : b3::IV[i];
    const u64* p = enc + (size_t)r0 * nn + col;
    for (u32 b = 0; b < nb; b++) {
        uint32_t m[16];
        const u32 cnt = min(8u, r1 - r0 - 8u * b);
#pragma unroll
        for (u32 i = 0; i < 8; i++) {
            u64 w = i < cnt ? p[(size_t)(8u * b + i) * nn] : 0ull;
            m[2 * i] = (uint32_t)w;
            m[2 * i + 1] = (uint32_t)(w >> 32);
        }
        uint32_t flags = mode | (b == 0 ? b3::CHUNK_START : 0u);
        if (b == nb - 1) flags |= b3::CHUNK_END | (nchunks == 1 ? b3::ROOT : 0u);
        b3::compress(cv, m, chunk, cnt * 8u, flags);
    }
    uint32_t* dst = nchunks == 1 ? leaves + (size_t)col * 8 : cvs + ((size_t)chunk * nn + col) * 8;
#pragma unroll
    for (int i = 0; i < 8; i++) dst[i] = cv[i];
}

// pass 2: join a column's chunk values along BLAKE3's tree (complete power-of-two subtrees first,
// the remainder from the right, ROOT on the last join)
__global__ void __launch_bounds__(128) k_static_col_merge(const uint32_t* __restrict__ cvs, u32 nn, u32 nchunks, Key8 key,
                                                          uint32_t* __restrict__ leaves) {
    const u32 col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= nn) return;
    uint32_t stack[24][8];
    int sp = 0;
    auto join = [&](bool root) {
        uint32_t m[16], out[8];
#pragma unroll
        for (int i = 0; i < 8; i++) { m[i] = stack[sp - 2][i]; m[8 + i] = stack[sp - 1][i]; out[i] = key.keyed ? key.w[i] : b3::IV[i]; }
        b3::compress(out, m, 0, 64, b3::PARENT | (key.keyed ? b3::KEYED : 0u) | (root ? b3::ROOT : 0u));
        sp--;
#pragma unroll
        for (int i = 0; i < 8; i++) stack[sp - 1][i] = out[i];
    };
    for (u32 c = 0; c < nchunks; c++) {
        const uint32_t* src = cvs + ((size_t)c * nn + col) * 8;
#pragma unroll
        for (int i = 0; i < 8; i++) stack[sp][i] = src[i];
        sp++;
        if (c + 1 == nchunks) break;
        for (u32 t = c + 1; (t & 1u) == 0; t >>= 1) join(false);
    }
    while (sp > 1) join(sp == 2);
    uint32_t* dst = leaves + (size_t)col * 8;
#pragma unroll
    for (int i = 0; i < 8; i++) dst[i] = stack[0][i];
}

constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
void* g_cv_addr[MAX_DEVICES];  // per device: the array's device address, resolved on first use

}  // namespace

extern "C" int hl_b200_hash_columns_static(const uint64_t* d_encoded, size_t rows, size_t nn, const uint8_t* key32,
                                           uint8_t* d_leaves32, void* cuda_stream) {
    if (!d_encoded || !d_leaves32 || rows == 0 || nn == 0 || rows > 0x7FFFFFFFu || nn > 0x7FFFFFFFu) return HL_B200_ERR_ARG;
    if (((uintptr_t)d_encoded & 7) || ((uintptr_t)d_leaves32 & 3)) return HL_B200_ERR_ARG;  // words are loaded as u64, leaves stored as u32
    const size_t nchunks = (rows + 127) / 128;
    if (nchunks > 65535) return HL_B200_ERR_UNSUPPORTED;
    if (nchunks > 1 && nchunks * nn * 32 > (size_t)HL_B200_STATIC_CV_BYTES) return HL_B200_ERR_UNSUPPORTED;  // beyond the static scratch
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return HL_B200_ERR_DEVICE;
    void* cv = nullptr;
    {
        std::lock_guard<std::mutex> g(g_mu);
        if (!g_cv_addr[dev]) {
            void* p = nullptr;
            if (cudaGetSymbolAddress(&p, g_static_cv) != cudaSuccess || !p) {
                cudaGetLastError();
                return HL_B200_ERR_DEVICE;
            }
            g_cv_addr[dev] = p;
        }
        cv = g_cv_addr[dev];
    }
    Key8 key{};
    key.keyed = key32 ? 1 : 0;
    if (key32)
        for (int i = 0; i < 8; i++)
            key.w[i] = (uint32_t)key32[4 * i] | ((uint32_t)key32[4 * i + 1] << 8) | ((uint32_t)key32[4 * i + 2] << 16) | ((uint32_t)key32[4 * i + 3] << 24);
    cudaStream_t st = (cudaStream_t)cuda_stream;
    dim3 grid((unsigned)((nn + 127) / 128), (unsigned)nchunks);
    k_static_col_chunks<<<grid, 128, 0, st>>>((const u64*)d_encoded, (u32)rows, (u32)nn, key, (u32)nchunks, (uint32_t*)cv, (uint32_t*)d_leaves32);
    if (cudaGetLastError() != cudaSuccess) return HL_B200_ERR_DEVICE;
    if (nchunks > 1) {
        k_static_col_merge<<<(unsigned)((nn + 127) / 128), 128, 0, st>>>((const uint32_t*)cv, (u32)nn, (u32)nchunks, key, (uint32_t*)d_leaves32);
        if (cudaGetLastError() != cudaSuccess) return HL_B200_ERR_DEVICE;
    }
    return HL_B200_OK;
}
