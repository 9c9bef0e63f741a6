// The prover's random stream expanded on the device (zkp-core/src/rng.rs:279-417 ZkRng).
//
// The stream is BLAKE3 in counter mode: block c is the first 8,192 extended-output bytes of H(key || LE64(c)), the blocks
// are concatenated, consecutive little-endian u64 words are the draws; fp() takes two words (low one first) and
// reduces the 128-bit value mod p (rng.rs:306-332), fill_fp is that loop (rng.rs:354-404), bytes32 is four words
// (rng.rs:410-416).  Every 64-byte piece of extended output is ONE compression of the same 40-byte message with its
// own output counter, so the pieces are independent: one thread per piece.
//
// The backend draws no randomness of its own (pcs/backend.rs:11-16): key and stream position stay with the caller's
// generator, which skips the words it had expanded here.  What this removes is the host-serial draw of a hiding
// commitment's pads and salts (pcs.rs:733-745, 788-792: 11 MB of stream per 8B `A` commitment).
#include "api_internal.h"
#include "b3.cuh"
#include "gl_field.cuh"

using namespace hlapi;

namespace {

// words [first, first + count) of the stream; thread t produces the 8 words of piece first/8 + t
__global__ void __launch_bounds__(128) k_rng_words(const uint32_t* __restrict__ key, u64 first, u64 count, u64* __restrict__ out) {
    const u64 piece = first / 8 + (u64)blockIdx.x * blockDim.x + threadIdx.x;
    if (piece * 8 >= first + count) return;
    const u64 block = piece / 128;           // 8,192 bytes = 128 pieces of 64 bytes
    const u64 t = piece % 128;               // the piece's output counter inside its block
    uint32_t m[16], v[16];
#pragma unroll
    for (int i = 0; i < 8; i++) m[i] = key[i];
    m[8] = (uint32_t)block; m[9] = (uint32_t)(block >> 32);
#pragma unroll
    for (int i = 10; i < 16; i++) m[i] = 0;
    b3::compress_xof(v, b3::IV, m, t, 40, b3::CHUNK_START | b3::CHUNK_END | b3::ROOT);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const u64 w = piece * 8 + i;
        if (w >= first && w < first + count) out[w - first] = ((u64)v[2 * i + 1] << 32) | v[2 * i];
    }
}

// out[k] = (words[2k] + 2^64 words[2k+1]) mod p
__global__ void __launch_bounds__(256) k_rng_fp(const u64* __restrict__ words, u64 n, u64* __restrict__ out) {
    const u64 k = (u64)blockIdx.x * blockDim.x + threadIdx.x;
    if (k < n) out[k] = gl_reduce128(words[2 * k], words[2 * k + 1]);
}

int launch_words(hl_ctx* c, const uint32_t* d_key, u64 first, u64 count, u64* d_out) {
    const u64 pieces = (first + count + 7) / 8 - first / 8;
    k_rng_words<<<(unsigned)((pieces + 127) / 128), 128, 0, c->stream>>>(d_key, first, count, d_out);
    c->stats.kernel_launches++;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? HL_B200_OK : fail(c, HL_B200_ERR_DEVICE, "rng launch", e);
}

// words (as_fp == 0) or field elements (as_fp != 0) of the stream into device memory
int fill_dev(hl_ctx* c, const uint8_t* key32, u64 first_word, u64 count, int as_fp, u64* d_out) {
    if (count == 0) return HL_B200_OK;
    if (count > ((u64)1 << 34) || first_word > ((u64)1 << 60)) return fail(c, HL_B200_ERR_ARG, "rng: range");
    uint32_t* d_key = nullptr;
    int rc = upload_key(c, key32, &d_key);
    u64* d_words = nullptr;
    const u64 nw = as_fp ? 2 * count : count;
    if (!rc && as_fp) rc = dev_alloc(c, (void**)&d_words, nw * 8);
    if (!rc) rc = launch_words(c, d_key, first_word, nw, as_fp ? d_words : d_out);
    if (!rc && as_fp) {
        k_rng_fp<<<(unsigned)((count + 255) / 256), 256, 0, c->stream>>>(d_words, count, d_out);
        c->stats.kernel_launches++;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "rng reduce launch", e);
    }
    if (d_words) dev_free(c, d_words, nw * 8);
    if (d_key) dev_free(c, d_key, 32);
    return rc;
}

}  // namespace

extern "C" {

int hl_b200_rng_fill_dev(hl_ctx* c, const uint8_t* key32, uint64_t first_word, uint64_t count, int as_fp, uint64_t* d_out) {
    if (!c || !key32 || (count && !d_out)) return fail(c, HL_B200_ERR_ARG, "rng_fill_dev: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    return fill_dev(c, key32, first_word, count, as_fp, reinterpret_cast<u64*>(d_out));
}

int hl_b200_rng_fill(hl_ctx* c, const uint8_t* key32, uint64_t first_word, uint64_t count, int as_fp, uint64_t* out) {
    if (!c || !key32 || (count && !out)) return fail(c, HL_B200_ERR_ARG, "rng_fill: null argument");
    if (count == 0) return HL_B200_OK;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    u64* d_out = nullptr;
    int rc = dev_alloc(c, (void**)&d_out, count * 8);
    if (!rc) rc = fill_dev(c, key32, first_word, count, as_fp, d_out);
    if (!rc) rc = d2h(c, out, d_out, count * 8);
    if (!rc) rc = sync(c, "rng_fill");
    if (d_out) dev_free(c, d_out, count * 8);
    return rc;
}

}  // extern "C"
