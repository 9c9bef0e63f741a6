/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * CPU restatement of the reference prover's Goldilocks field, used only as the
 * checker in tests, the smoke check and the CPU-baseline leg of the bench.
 *
 * Follows zkp-core/src/field.rs:10-239 (ops/zkp-mvp/gpu-metal tree):
 *   p = 2^64 - 2^32 + 1, every stored word canonical (< p);
 *   Fp2 = Fp[u]/(u^2 - 7), element (c0, c1), bytes LE(c0) || LE(c1).
 */
#ifndef HL_ORACLE_FIELD_H
#define HL_ORACLE_FIELD_H
#include <stdint.h>
#include <stddef.h>

#define OR_P 0xFFFFFFFF00000001ULL
#define OR_EPS 0xFFFFFFFFULL

typedef unsigned __int128 u128;
typedef struct { uint64_t c0, c1; } fp2_t;

/* field.rs:27-29 */
static inline uint64_t fp_new(uint64_t v) { return v >= OR_P ? v - OR_P : v; }

/* field.rs:103-116 (reduce128): exact for every 128-bit input */
static inline uint64_t fp_reduce128(u128 x) {
    uint64_t lo = (uint64_t)x, hi = (uint64_t)(x >> 64);
    uint64_t hh = hi >> 32, hl = hi & OR_EPS;
    uint64_t t0 = lo - hh;
    if (lo < hh) t0 -= OR_EPS;
    uint64_t t1 = hl * OR_EPS;
    uint64_t r = t0 + t1;
    if (r < t0) r += OR_EPS;
    return fp_new(r);
}
/* field.rs:45-49 */
static inline uint64_t fp_add(uint64_t a, uint64_t b) {
    uint64_t r = a + b;
    if (r < a) r += OR_EPS;
    return fp_new(r);
}
/* field.rs:51-54 */
static inline uint64_t fp_sub(uint64_t a, uint64_t b) {
    uint64_t r = a - b;
    if (a < b) r -= OR_EPS;
    return r;
}
static inline uint64_t fp_neg(uint64_t a) { return a ? OR_P - a : 0; }
static inline uint64_t fp_mul(uint64_t a, uint64_t b) { return fp_reduce128((u128)a * b); }
/* field.rs:32-34 */
static inline uint64_t fp_from_i64(int64_t v) {
    if (v >= 0) return fp_new((uint64_t)v);
    uint64_t m = (uint64_t)(-(v + 1)) + 1; /* |v| without overflow */
    return fp_new(OR_P - m % OR_P);
}
static inline uint64_t fp_pow(uint64_t b, uint64_t e) {
    uint64_t acc = 1;
    while (e) { if (e & 1) acc = fp_mul(acc, b); b = fp_mul(b, b); e >>= 1; }
    return acc;
}
static inline uint64_t fp_inv(uint64_t a) { return fp_pow(a, OR_P - 2); }
/* field.rs:86-91 */
static inline uint64_t fp_two_adic_root(uint32_t k) {
    uint64_t r32 = fp_pow(7, (OR_P - 1) >> 32);
    return fp_pow(r32, 1ULL << (32 - k));
}

static inline fp2_t fp2_new(uint64_t a, uint64_t b) { fp2_t r = {a, b}; return r; }
static inline fp2_t fp2_add(fp2_t a, fp2_t b) { return fp2_new(fp_add(a.c0, b.c0), fp_add(a.c1, b.c1)); }
static inline fp2_t fp2_sub(fp2_t a, fp2_t b) { return fp2_new(fp_sub(a.c0, b.c0), fp_sub(a.c1, b.c1)); }
static inline fp2_t fp2_neg(fp2_t a) { return fp2_new(fp_neg(a.c0), fp_neg(a.c1)); }
/* field.rs:163-169 */
static inline fp2_t fp2_mul(fp2_t a, fp2_t b) {
    uint64_t ac = fp_mul(a.c0, b.c0), bd = fp_mul(a.c1, b.c1);
    uint64_t ad = fp_mul(a.c0, b.c1), bc = fp_mul(a.c1, b.c0);
    return fp2_new(fp_add(ac, fp_mul(bd, 7)), fp_add(ad, bc));
}
static inline fp2_t fp2_mul_base(fp2_t a, uint64_t b) { return fp2_new(fp_mul(a.c0, b), fp_mul(a.c1, b)); }
static inline int fp2_is_zero(fp2_t a) { return a.c0 == 0 && a.c1 == 0; }
static inline int fp2_eq(fp2_t a, fp2_t b) { return a.c0 == b.c0 && a.c1 == b.c1; }
/* field.rs:180-185 */
static inline fp2_t fp2_inv(fp2_t a) {
    uint64_t norm = fp_sub(fp_mul(a.c0, a.c0), fp_mul(fp_mul(a.c1, a.c1), 7));
    uint64_t ni = fp_inv(norm);
    return fp2_new(fp_mul(a.c0, ni), fp_mul(fp_neg(a.c1), ni));
}
static const fp2_t FP2_ZERO = {0, 0};
static const fp2_t FP2_ONE = {1, 0};

#endif
