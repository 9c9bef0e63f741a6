/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * CPU restatement of the reference's Fiat-Shamir transcript
 * (zkp-core/src/transcript.rs:29-167) and prover RNG (zkp-core/src/rng.rs:279-417).
 */
#include "hl_oracle.h"
#include <stdlib.h>
#include <string.h>

static void le64(uint64_t v, uint8_t *o) { for (int i = 0; i < 8; i++) o[i] = (uint8_t)(v >> (8 * i)); }
static uint64_t rd64(const uint8_t *p) { uint64_t v = 0; for (int i = 0; i < 8; i++) v |= (uint64_t)p[i] << (8 * i); return v; }

/* transcript.rs:29-45: state = H("hashline-v1/" || domain); keyed when a key is given */
void or_tr_new(or_transcript *t, const uint8_t *domain, size_t len, const uint8_t *key) {
    uint8_t *m = (uint8_t *)malloc(12 + len);
    memcpy(m, "hashline-v1/", 12);
    if (len) memcpy(m + 12, domain, len);
    t->keyed = key != NULL;
    if (key) memcpy(t->key, key, 32); else memset(t->key, 0, 32);
    or_blake3(key, m, 12 + len, t->state, 32);
    t->counter = 0;
    free(m);
}

/* transcript.rs:67-74: state' = H(state || LE64(|label|) || label || LE64(|data|) || data) */
void or_tr_absorb(or_transcript *t, const uint8_t *label, size_t llen, const uint8_t *data, size_t dlen) {
    size_t tot = 32 + 8 + llen + 8 + dlen;
    uint8_t *m = (uint8_t *)malloc(tot), *p = m;
    memcpy(p, t->state, 32); p += 32;
    le64(llen, p); p += 8;
    if (llen) memcpy(p, label, llen);
    p += llen;
    le64(dlen, p); p += 8;
    if (dlen) memcpy(p, data, dlen);
    or_blake3(t->keyed ? t->key : NULL, m, tot, t->state, 32);
    free(m);
}

/* transcript.rs:120-130: out = H(state || "squeeze" || LE64(counter)); counter++; state = out */
void or_tr_squeeze(or_transcript *t, uint8_t out[32]) {
    uint8_t m[47];
    memcpy(m, t->state, 32);
    memcpy(m + 32, "squeeze", 7);
    le64(t->counter, m + 39);
    t->counter++;
    or_blake3(t->keyed ? t->key : NULL, m, 47, out, 32);
    memcpy(t->state, out, 32);
}

static uint64_t fp_from_le16(const uint8_t *b) { return fp_reduce128(((u128)rd64(b + 8) << 64) | rd64(b)); }

/* transcript.rs:133-148 */
uint64_t or_tr_challenge_fp(or_transcript *t) {
    uint8_t b[32];
    or_tr_squeeze(t, b);
    return fp_from_le16(b);
}
void or_tr_challenge_fp2(or_transcript *t, uint64_t out[2]) {
    uint8_t b[32];
    or_tr_squeeze(t, b);
    out[0] = fp_from_le16(b);
    out[1] = fp_from_le16(b + 16);
}
/* transcript.rs:155-167: four LE u64 per squeeze, each masked with bound - 1 */
void or_tr_challenge_indices(or_transcript *t, size_t n, uint64_t bound, uint64_t *out) {
    size_t got = 0;
    while (got < n) {
        uint8_t b[32];
        or_tr_squeeze(t, b);
        for (int c = 0; c < 4 && got < n; c++) out[got++] = rd64(b + 8 * c) & (bound - 1);
    }
}

/* rng.rs:279-284: key = H("hashline-zk-rng/" || domain || LE64(seed)) */
void or_rng_new(or_rng *r, uint64_t seed, const uint8_t *domain, size_t len) {
    uint8_t *m = (uint8_t *)malloc(16 + len + 8);
    memcpy(m, "hashline-zk-rng/", 16);
    if (len) memcpy(m + 16, domain, len);
    le64(seed, m + 16 + len);
    or_blake3(NULL, m, 24 + len, r->key, 32);
    r->counter = 0;
    r->pos = sizeof r->buf;
    free(m);
}
/* rng.rs:25-30,306-310: block c = the first 8192 XOF bytes of H(key || LE64(c)) */
static void refill(or_rng *r) {
    uint8_t m[40];
    memcpy(m, r->key, 32);
    le64(r->counter, m + 32);
    or_blake3(NULL, m, 40, r->buf, sizeof r->buf);
    r->counter++;
    r->pos = 0;
}
uint64_t or_rng_next_u64(or_rng *r) {
    if (r->pos + 8 > sizeof r->buf) refill(r);
    uint64_t v = rd64(r->buf + r->pos);
    r->pos += 8;
    return v;
}
/* rng.rs:323-327: lo is drawn first, then hi */
uint64_t or_rng_fp(or_rng *r) {
    uint64_t lo = or_rng_next_u64(r), hi = or_rng_next_u64(r);
    return fp_reduce128(((u128)hi << 64) | lo);
}
/* rng.rs:354-404: word for word the fp() loop, including the state it leaves */
void or_rng_fill_fp(or_rng *r, uint64_t *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = or_rng_fp(r);
}
/* rng.rs:410-416 */
void or_rng_bytes32(or_rng *r, uint8_t out[32]) {
    for (int c = 0; c < 4; c++) le64(or_rng_next_u64(r), out + 8 * c);
}
