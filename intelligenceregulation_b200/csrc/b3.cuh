// BLAKE3 compression function for device code, written from the published
// specification.  The prover's hashes (column leaves pcs.rs:176-221, salted
// leaves pcs.rs:696-715, tree nodes merkle.rs:14-31, transcript
// transcript.rs:67-130) are BLAKE3 in its plain or keyed mode; keyed mode
// replaces the initial chaining value by the key words and sets one flag bit.
//
// All 16 state words and 16 message words stay in registers: the seven rounds
// are unrolled with the message schedule resolved at compile time.
#pragma once
#include <stdint.h>

namespace b3 {

enum : uint32_t { CHUNK_START = 1, CHUNK_END = 2, PARENT = 4, ROOT = 8, KEYED = 16 };

static __device__ __constant__ const uint32_t IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au,
                                                0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};

// sigma^r(i): which input word feeds slot i in round r (the message permutation applied r times)
__host__ __device__ constexpr int sched(int r, int i) {
    const int perm[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
    for (int k = 0; k < r; k++) i = perm[i];
    return i;
}

__device__ __forceinline__ uint32_t rotr(uint32_t x, int n) { return __funnelshift_r(x, x, n); }

__device__ __forceinline__ void g(uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d, uint32_t mx, uint32_t my) {
    a = a + b + mx;
    d = rotr(d ^ a, 16);
    c = c + d;
    b = rotr(b ^ c, 12);
    a = a + b + my;
    d = rotr(d ^ a, 8);
    c = c + d;
    b = rotr(b ^ c, 7);
}

template <int R, int I>
struct S {
    static constexpr int v = sched(R, I);
};

template <int R>
__device__ __forceinline__ void round_fn(uint32_t (&v)[16], const uint32_t (&m)[16]) {
    g(v[0], v[4], v[8], v[12], m[S<R, 0>::v], m[S<R, 1>::v]);
    g(v[1], v[5], v[9], v[13], m[S<R, 2>::v], m[S<R, 3>::v]);
    g(v[2], v[6], v[10], v[14], m[S<R, 4>::v], m[S<R, 5>::v]);
    g(v[3], v[7], v[11], v[15], m[S<R, 6>::v], m[S<R, 7>::v]);
    g(v[0], v[5], v[10], v[15], m[S<R, 8>::v], m[S<R, 9>::v]);
    g(v[1], v[6], v[11], v[12], m[S<R, 10>::v], m[S<R, 11>::v]);
    g(v[2], v[7], v[8], v[13], m[S<R, 12>::v], m[S<R, 13>::v]);
    g(v[3], v[4], v[9], v[14], m[S<R, 14>::v], m[S<R, 15>::v]);
}

// cv <- first eight output words of compress(cv, m, counter, block_len, flags)
__device__ __forceinline__ void compress(uint32_t (&cv)[8], const uint32_t (&m)[16], uint64_t counter,
                                         uint32_t block_len, uint32_t flags) {
    uint32_t v[16];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = cv[i];
    v[8] = 0x6A09E667u; v[9] = 0xBB67AE85u; v[10] = 0x3C6EF372u; v[11] = 0xA54FF53Au;
    v[12] = (uint32_t)counter; v[13] = (uint32_t)(counter >> 32);
    v[14] = block_len; v[15] = flags;
    round_fn<0>(v, m); round_fn<1>(v, m); round_fn<2>(v, m); round_fn<3>(v, m);
    round_fn<4>(v, m); round_fn<5>(v, m); round_fn<6>(v, m);
#pragma unroll
    for (int i = 0; i < 8; i++) cv[i] = v[i] ^ v[i + 8];
}

// all sixteen output words of compress(cv, m, counter, block_len, flags): the extended output of a root node, whose
// counter is the index of the 64-byte output piece
__device__ __forceinline__ void compress_xof(uint32_t (&out)[16], const uint32_t* cv, const uint32_t (&m)[16], uint64_t counter,
                                             uint32_t block_len, uint32_t flags) {
    uint32_t v[16];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = cv[i];
    v[8] = 0x6A09E667u; v[9] = 0xBB67AE85u; v[10] = 0x3C6EF372u; v[11] = 0xA54FF53Au;
    v[12] = (uint32_t)counter; v[13] = (uint32_t)(counter >> 32);
    v[14] = block_len; v[15] = flags;
    round_fn<0>(v, m); round_fn<1>(v, m); round_fn<2>(v, m); round_fn<3>(v, m);
    round_fn<4>(v, m); round_fn<5>(v, m); round_fn<6>(v, m);
#pragma unroll
    for (int i = 0; i < 8; i++) { out[i] = v[i] ^ v[i + 8]; out[i + 8] = v[i + 8] ^ cv[i]; }
}

// start-of-hash chaining value: the IV, or the key words in keyed mode
__device__ __forceinline__ void init_cv(uint32_t (&cv)[8], const uint32_t* key) {
#pragma unroll
    for (int i = 0; i < 8; i++) cv[i] = key ? key[i] : IV[i];
}

// digest of a 64-byte message (one chunk, one block): salted leaves and tree nodes
__device__ __forceinline__ void hash64(uint32_t (&out)[8], const uint32_t (&m)[16], const uint32_t* key) {
    init_cv(out, key);
    compress(out, m, 0, 64, CHUNK_START | CHUNK_END | ROOT | (key ? KEYED : 0u));
}

}  // namespace b3
