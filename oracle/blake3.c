/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * A plain restatement of the published BLAKE3 algorithm (hash, keyed hash,
 * derive_key, extendable output) for whole in-memory messages.
 *
 * The reference prover takes BLAKE3 from the third-party crate `blake3`
 * (pinned 1.8.7 in hashline/Cargo.lock and zkp-core/Cargo.lock), which is not
 * part of the reference tree.  Its call sites are zkp-core/src/merkle.rs:15-31,
 * pcs.rs:158-220,697-714, hashtag.rs:95-98,154-158, transcript.rs:30-33,68-74,
 * 122-128 and rng.rs:25-30,280-284.  This file is pinned against the `B3`
 * records of the reference's L5 agreement corpus (hash / keyed / derive at 37
 * lengths) and the eight derived hash-tag keys of hashtag.rs:188-198.
 *
 * Shape of this implementation: a recursive walk of the chunk tree over a
 * contiguous buffer.  A subtree of more than one chunk splits at the largest
 * power-of-two number of chunks strictly below its size; the two chaining
 * values are joined by a parent compression; the outermost compression
 * carries the ROOT flag and, for extendable output, the output-block counter.
 */
#include "hl_oracle.h"
#include <string.h>

enum { F_CHUNK_START = 1, F_CHUNK_END = 2, F_PARENT = 4, F_ROOT = 8,
       F_KEYED = 16, F_DERIVE_CTX = 32, F_DERIVE_MAT = 64 };

static const uint32_t B3_IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au,
                                  0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
static const uint8_t B3_PERM[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};

static inline uint32_t ror(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

#define QR(a, b, c, d, x, y)                                   \
    do {                                                       \
        v[a] += v[b] + (x); v[d] = ror(v[d] ^ v[a], 16);       \
        v[c] += v[d];       v[b] = ror(v[b] ^ v[c], 12);       \
        v[a] += v[b] + (y); v[d] = ror(v[d] ^ v[a], 8);        \
        v[c] += v[d];       v[b] = ror(v[b] ^ v[c], 7);        \
    } while (0)

/* One compression; writes all 16 output words (the first 8 are the new
 * chaining value, all 16 are one extendable-output block). */
static void compress(const uint32_t cv[8], const uint32_t block[16], uint64_t counter,
                     uint32_t block_len, uint32_t flags, uint32_t out[16]) {
    uint32_t v[16], m[16], t[16];
    for (int i = 0; i < 8; i++) v[i] = cv[i];
    for (int i = 0; i < 4; i++) v[8 + i] = B3_IV[i];
    v[12] = (uint32_t)counter; v[13] = (uint32_t)(counter >> 32);
    v[14] = block_len; v[15] = flags;
    memcpy(m, block, 64);
    for (int r = 0; r < 7; r++) {
        QR(0, 4, 8, 12, m[0], m[1]);   QR(1, 5, 9, 13, m[2], m[3]);
        QR(2, 6, 10, 14, m[4], m[5]);  QR(3, 7, 11, 15, m[6], m[7]);
        QR(0, 5, 10, 15, m[8], m[9]);  QR(1, 6, 11, 12, m[10], m[11]);
        QR(2, 7, 8, 13, m[12], m[13]); QR(3, 4, 9, 14, m[14], m[15]);
        for (int i = 0; i < 16; i++) t[i] = m[B3_PERM[i]];
        memcpy(m, t, 64);
    }
    for (int i = 0; i < 8; i++) { out[i] = v[i] ^ v[i + 8]; out[i + 8] = v[i + 8] ^ cv[i]; }
}

static void load_block(const uint8_t *p, size_t len, uint32_t w[16]) {
    uint8_t b[64];
    memset(b, 0, 64);
    if (len) memcpy(b, p, len);
    for (int i = 0; i < 16; i++)
        w[i] = (uint32_t)b[4 * i] | ((uint32_t)b[4 * i + 1] << 8) | ((uint32_t)b[4 * i + 2] << 16) | ((uint32_t)b[4 * i + 3] << 24);
}

/* What the LAST compression of a subtree needs, so that the caller can decide
 * whether it is the root. */
typedef struct { uint32_t cv[8]; uint32_t block[16]; uint64_t counter; uint32_t block_len, flags; } tail_t;

/* Hash one chunk (<= 1024 bytes) up to, but not including, its last block. */
static void chunk_tail(const uint32_t key[8], uint32_t mode, const uint8_t *p, size_t len, uint64_t chunk_idx, tail_t *t) {
    uint32_t cv[8], out[16], w[16];
    memcpy(cv, key, 32);
    size_t nblocks = len ? (len + 63) / 64 : 1;
    for (size_t b = 0; b + 1 < nblocks; b++) {
        load_block(p + 64 * b, 64, w);
        compress(cv, w, chunk_idx, 64, mode | (b == 0 ? F_CHUNK_START : 0), out);
        memcpy(cv, out, 32);
    }
    size_t last = nblocks - 1, llen = len - 64 * last;
    memcpy(t->cv, cv, 32);
    load_block(p + 64 * last, llen, t->block);
    t->counter = chunk_idx;
    t->block_len = (uint32_t)llen;
    t->flags = mode | (last == 0 ? F_CHUNK_START : 0) | F_CHUNK_END;
}

static void subtree_tail(const uint32_t key[8], uint32_t mode, const uint8_t *p, size_t len, uint64_t chunk0, tail_t *t);

static void subtree_cv(const uint32_t key[8], uint32_t mode, const uint8_t *p, size_t len, uint64_t chunk0, uint32_t cv[8]) {
    tail_t t;
    uint32_t out[16];
    subtree_tail(key, mode, p, len, chunk0, &t);
    compress(t.cv, t.block, t.counter, t.block_len, t.flags, out);
    memcpy(cv, out, 32);
}

static void subtree_tail(const uint32_t key[8], uint32_t mode, const uint8_t *p, size_t len, uint64_t chunk0, tail_t *t) {
    if (len <= 1024) { chunk_tail(key, mode, p, len, chunk0, t); return; }
    /* left side: the largest power-of-two count of whole chunks strictly below len */
    size_t chunks = (len - 1) / 1024, left = 1;
    while (left * 2 <= chunks) left *= 2;
    subtree_cv(key, mode, p, left * 1024, chunk0, t->block);
    subtree_cv(key, mode, p + left * 1024, len - left * 1024, chunk0 + left, t->block + 8);
    memcpy(t->cv, key, 32);
    t->counter = 0; t->block_len = 64; t->flags = mode | F_PARENT;
}

static void hash_mode(const uint32_t key[8], uint32_t mode, const uint8_t *data, size_t len, uint8_t *out, size_t outlen) {
    tail_t t;
    uint32_t w[16];
    subtree_tail(key, mode, data, len, 0, &t);
    for (uint64_t blk = 0; blk * 64 < outlen; blk++) {
        compress(t.cv, t.block, blk, t.block_len, t.flags | F_ROOT, w);
        size_t take = outlen - blk * 64 < 64 ? outlen - blk * 64 : 64;
        for (size_t i = 0; i < take; i++) out[blk * 64 + i] = (uint8_t)(w[i / 4] >> (8 * (i % 4)));
    }
}

static void key_words(const uint8_t key[32], uint32_t w[8]) {
    for (int i = 0; i < 8; i++)
        w[i] = (uint32_t)key[4 * i] | ((uint32_t)key[4 * i + 1] << 8) | ((uint32_t)key[4 * i + 2] << 16) | ((uint32_t)key[4 * i + 3] << 24);
}

/* key == NULL: the unkeyed hash; otherwise BLAKE3's keyed mode.  `outlen`
 * bytes of (extendable) output. */
void or_blake3(const uint8_t *key, const uint8_t *data, size_t len, uint8_t *out, size_t outlen) {
    uint32_t kw[8];
    if (key) { key_words(key, kw); hash_mode(kw, F_KEYED, data, len, out, outlen); }
    else hash_mode(B3_IV, 0, data, len, out, outlen);
}

void or_blake3_derive_key(const uint8_t *context, size_t ctx_len, const uint8_t *material, size_t len, uint8_t out[32]) {
    uint8_t ck[32];
    uint32_t kw[8];
    hash_mode(B3_IV, F_DERIVE_CTX, context, ctx_len, ck, 32);
    key_words(ck, kw);
    hash_mode(kw, F_DERIVE_MAT, material, len, out, 32);
}
