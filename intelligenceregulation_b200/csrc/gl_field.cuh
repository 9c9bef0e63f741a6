// Goldilocks field arithmetic for device (and host) code.
//
// p = 2^64 - 2^32 + 1.  Every value handed to or returned from these functions
// is canonical (< p), which is the representation the reference prover keeps
// (zkp-core/src/field.rs:10-116).  The extension is Fp2 = Fp[u]/(u^2 - 7),
// stored as two consecutive words (c0, c1) (field.rs:139-203).
//
// The reduction uses 2^64 = 2^32 - 1 and 2^96 = -1 (mod p): a 128-bit product
// lo + 2^64 (hh 2^32 + hl) equals lo - hh + hl (2^32 - 1).  No division, no
// Montgomery form: canonical words go straight to the BLAKE3 column hash.
#pragma once
#include <stdint.h>

#ifdef __CUDACC__
#define GL_HD __host__ __device__ __forceinline__
#define GL_HDC __host__ __device__ constexpr
#else
#define GL_HD inline
#define GL_HDC constexpr
#endif

typedef unsigned long long u64;
typedef unsigned int u32;

#define GL_P 0xFFFFFFFF00000001ULL
#define GL_EPS 0xFFFFFFFFULL

struct fp2 {
    u64 c0, c1;
};

GL_HD u64 gl_canon(u64 v) { return v >= GL_P ? v - GL_P : v; }

// ---- lazy forms for butterfly chains -------------------------------------------------------------
// A "lazy" word is any u64 congruent to the value mod p (canonical or not).  Inside the NTT passes the
// elements stay lazy and only products are brought back to canonical form, which is what lets every
// add / sub get by with ONE conditional correction:
//   gl_mul_lazy(a, b)   any a, b            -> lazy product
//   gl_add_lazy(u, v)   u lazy, v CANONICAL -> lazy sum        (u + v < 2^65 - 2^32 + 1: one wrap at most)
//   gl_sub_lazy(u, v)   u lazy, v CANONICAL -> lazy difference (u - v + 2^64 >= 2^32 - 1: one borrow at most)
// On the device they are PTX carry chains over 32-bit limbs (the 64-bit C forms cost ~1.5x the ALU-pipe
// instructions); the multiply builds the 128-bit product with four 32x32 multiply-adds.
#ifdef __CUDA_ARCH__
__device__ __forceinline__ u64 gl_mul_lazy(u64 a, u64 b) {
    const u32 a0 = (u32)a, a1 = (u32)(a >> 32), b0 = (u32)b, b1 = (u32)(b >> 32);
    const u64 x = (u64)a0 * b0;
    const u64 y = (u64)a0 * b1 + (x >> 32);
    const u64 z = (u64)a1 * b0 + (u32)y;
    const u64 w = (u64)a1 * b1 + (y >> 32) + (z >> 32);
    const u32 p0 = (u32)x, p1 = (u32)z, p2 = (u32)w, p3 = (u32)(w >> 32);
    u32 r0, r1;
    // (p1:p0) - p3 [borrow: - EPS]  + p2 * EPS [carry: + EPS]
    asm("{\n\t"
        ".reg .u32 t0,t1,m,q0,q1;\n\t"
        ".reg .u64 q;\n\t"
        "sub.cc.u32 t0, %2, %5;\n\t"
        "subc.cc.u32 t1, %3, 0;\n\t"
        "subc.u32 m, 0, 0;\n\t"
        "sub.cc.u32 t0, t0, m;\n\t"
        "subc.u32 t1, t1, 0;\n\t"
        "mul.wide.u32 q, %4, 0xFFFFFFFF;\n\t"
        "mov.b64 {q0,q1}, q;\n\t"
        "add.cc.u32 t0, t0, q0;\n\t"
        "addc.cc.u32 t1, t1, q1;\n\t"
        "addc.u32 m, 0, 0;\n\t"
        "mov.b64 q, {t0,t1};\n\t"
        "mad.wide.u32 q, m, 0xFFFFFFFF, q;\n\t"
        "mov.b64 {%0,%1}, q;\n\t"
        "}"
        : "=r"(r0), "=r"(r1)
        : "r"(p0), "r"(p1), "r"(p2), "r"(p3));
    return ((u64)r1 << 32) | r0;
}
// r >= p  <=>  high limb all ones and low limb non-zero; then r - p = low limb - 1
__device__ __forceinline__ u64 gl_canon_fast(u64 r) {
    const u32 r0 = (u32)r, r1 = (u32)(r >> 32);
    return (r1 == 0xFFFFFFFFu && r0 != 0) ? (u64)(r0 - 1) : r;
}
__device__ __forceinline__ u64 gl_add_lazy(u64 u, u64 v) {
    const u32 u0 = (u32)u, u1 = (u32)(u >> 32), v0 = (u32)v, v1 = (u32)(v >> 32);
    u32 r0, r1;
    asm("{\n\t.reg .u32 m;\n\t.reg .u64 q;\n\t"
        "add.cc.u32 %0, %2, %4;\n\t"
        "addc.cc.u32 %1, %3, %5;\n\t"
        "addc.u32 m, 0, 0;\n\t"
        "mov.b64 q, {%0,%1};\n\t"
        "mad.wide.u32 q, m, 0xFFFFFFFF, q;\n\t"
        "mov.b64 {%0,%1}, q;\n\t}"
        : "=&r"(r0), "=&r"(r1) : "r"(u0), "r"(u1), "r"(v0), "r"(v1));
    return ((u64)r1 << 32) | r0;
}
__device__ __forceinline__ u64 gl_sub_lazy(u64 u, u64 v) {
    const u32 u0 = (u32)u, u1 = (u32)(u >> 32), v0 = (u32)v, v1 = (u32)(v >> 32);
    u32 r0, r1;
    asm("{\n\t.reg .u32 m;\n\t"
        "sub.cc.u32 %0, %2, %4;\n\t"
        "subc.cc.u32 %1, %3, %5;\n\t"
        "subc.u32 m, 0, 0;\n\t"
        "sub.cc.u32 %0, %0, m;\n\t"
        "subc.u32 %1, %1, 0;\n\t}"
        : "=&r"(r0), "=&r"(r1) : "r"(u0), "r"(u1), "r"(v0), "r"(v1));
    return ((u64)r1 << 32) | r0;
}
#else
// host forms with the same contracts (the phase emulation on the CPU runs these)
inline u64 gl_mul_lazy(u64 a, u64 b) {
    unsigned __int128 x = (unsigned __int128)a * b;
    u64 lo = (u64)x, hi = (u64)(x >> 64), hh = hi >> 32, hl = hi & GL_EPS;
    u64 t0 = lo - hh;
    if (lo < hh) t0 -= GL_EPS;
    u64 t1 = (hl << 32) - hl, r = t0 + t1;
    if (r < t0) r += GL_EPS;
    return r;  // not canonicalised
}
inline u64 gl_canon_fast(u64 r) { return gl_canon(r); }
inline u64 gl_add_lazy(u64 u, u64 v) {
    u64 r = u + v;
    if (r < u) r += GL_EPS;
    return r;
}
inline u64 gl_sub_lazy(u64 u, u64 v) {
    u64 r = u - v;
    if (u < v) r -= GL_EPS;
    return r;
}
#endif

// ---- canonical forms ----------------------------------------------------------------------------
// A translation unit tuned around the 64-bit C forms (the row encoder: its passes use the lazy forms directly, and its register
// allocation at 1,024 threads x 64 registers sits on the C forms of the few canonical operations around them; with the chains it
// measured 5 % slower) defines GL_PLAIN_CANONICAL_FORMS before this header and keeps them.
#if defined(__CUDA_ARCH__) && !defined(GL_PLAIN_CANONICAL_FORMS)
#define GL_DEVICE_CHAINS 1
#endif
// On the device they go through the carry chains above: measured on B200 with 32 resident warps, a dependent chain of each op,
// against the 64-bit C forms: add 1.19x, sub 1.68x, multiply 1.19x, Fp2 multiply 1.38x the throughput (the integer pipe issues a
// warp instruction every other cycle, so the instruction count is what counts).
GL_HD u64 gl_add(u64 a, u64 b) {
#ifdef GL_DEVICE_CHAINS
    return gl_canon_fast(gl_add_lazy(a, b));
#else
    u64 r = a + b;
    if (r < a) r += GL_EPS;  // wrapped past 2^64: 2^64 = EPS (mod p); the sum is then already < p
    return gl_canon(r);
#endif
}

GL_HD u64 gl_sub(u64 a, u64 b) {
#ifdef GL_DEVICE_CHAINS
    return gl_sub_lazy(a, b);  // canonical operands: a - b + p < p after the one borrow
#else
    u64 r = a - b;
    if (a < b) r -= GL_EPS;  // borrowed 2^64: give back EPS, i.e. add p
    return r;
#endif
}

GL_HD u64 gl_neg(u64 a) { return a ? GL_P - a : 0; }

#ifdef __CUDA_ARCH__
// (s3:s2:s1:s0) + c 2^128 as a lazy word: (s1:s0) - s3 - c 2^32 + s2 (2^32 - 1)   (2^96 = -1, 2^128 = -2^32 mod p)
__device__ __forceinline__ u64 gl_red129_lazy(u32 s0, u32 s1, u32 s2, u32 s3, u32 c) {
    u32 r0, r1;
    asm("{\n\t"
        ".reg .u32 t0,t1,m,q0,q1;\n\t"
        ".reg .u64 q;\n\t"
        "sub.cc.u32 t0, %2, %5;\n\t"
        "subc.cc.u32 t1, %3, %6;\n\t"
        "subc.u32 m, 0, 0;\n\t"
        "sub.cc.u32 t0, t0, m;\n\t"
        "subc.u32 t1, t1, 0;\n\t"
        "mul.wide.u32 q, %4, 0xFFFFFFFF;\n\t"
        "mov.b64 {q0,q1}, q;\n\t"
        "add.cc.u32 t0, t0, q0;\n\t"
        "addc.cc.u32 t1, t1, q1;\n\t"
        "addc.u32 m, 0, 0;\n\t"
        "mov.b64 q, {t0,t1};\n\t"
        "mad.wide.u32 q, m, 0xFFFFFFFF, q;\n\t"
        "mov.b64 {%0,%1}, q;\n\t"
        "}"
        : "=r"(r0), "=r"(r1)
        : "r"(s0), "r"(s1), "r"(s2), "r"(s3), "r"(c));
    return ((u64)r1 << 32) | r0;
}
#endif

GL_HD u64 gl_reduce128(u64 lo, u64 hi) {
#ifdef GL_DEVICE_CHAINS
    return gl_canon_fast(gl_red129_lazy((u32)lo, (u32)(lo >> 32), (u32)hi, (u32)(hi >> 32), 0u));
#else
    u64 hh = hi >> 32, hl = hi & GL_EPS;
    u64 t0 = lo - hh;
    if (lo < hh) t0 -= GL_EPS;
    u64 t1 = (hl << 32) - hl;  // hl * (2^32 - 1), below 2^64
    u64 r = t0 + t1;
    if (r < t0) r += GL_EPS;
    return gl_canon(r);
#endif
}

// the 128-bit product as (lo, hi); on the device four 32x32 multiply-adds into 64-bit accumulators
struct gl_wide {
    u64 lo, hi;
};
GL_HD gl_wide gl_mulw(u64 a, u64 b) {
    gl_wide r;
#ifdef __CUDA_ARCH__
    const u32 a0 = (u32)a, a1 = (u32)(a >> 32), b0 = (u32)b, b1 = (u32)(b >> 32);
    const u64 x = (u64)a0 * b0;
    const u64 y = (u64)a0 * b1 + (x >> 32);
    const u64 z = (u64)a1 * b0 + (u32)y;
    const u64 w = (u64)a1 * b1 + (y >> 32) + (z >> 32);
    r.lo = (z << 32) | (u32)x;
    r.hi = w;
#else
    unsigned __int128 x = (unsigned __int128)a * b;
    r.lo = (u64)x;
    r.hi = (u64)(x >> 64);
#endif
    return r;
}

GL_HD u64 gl_mul(u64 a, u64 b) {
#ifdef GL_DEVICE_CHAINS
    return gl_canon_fast(gl_mul_lazy(a, b));
#else
    const gl_wide w = gl_mulw(a, b);
    return gl_reduce128(w.lo, w.hi);
#endif
}


// a b + c d with ONE reduction: the 129-bit sum's top bit weighs 2^128 = -2^32 (mod p).  Device: any a, b, c, d (lazy operands too).
GL_HD u64 gl_mul_add2(u64 a, u64 b, u64 c, u64 d) {
    const gl_wide p = gl_mulw(a, b), q = gl_mulw(c, d);
#ifdef GL_DEVICE_CHAINS
    u32 s0, s1, s2, s3, cy;
    asm("add.cc.u32 %0, %5, %9;\n\taddc.cc.u32 %1, %6, %10;\n\taddc.cc.u32 %2, %7, %11;\n\taddc.cc.u32 %3, %8, %12;\n\taddc.u32 %4, 0, 0;"
        : "=r"(s0), "=r"(s1), "=r"(s2), "=r"(s3), "=r"(cy)
        : "r"((u32)p.lo), "r"((u32)(p.lo >> 32)), "r"((u32)p.hi), "r"((u32)(p.hi >> 32)), "r"((u32)q.lo), "r"((u32)(q.lo >> 32)), "r"((u32)q.hi),
          "r"((u32)(q.hi >> 32)));
    return gl_canon_fast(gl_red129_lazy(s0, s1, s2, s3, cy));
#else
    const u64 lo = p.lo + q.lo, cy = lo < p.lo ? 1u : 0u;
    const u64 h0 = p.hi + q.hi, c2 = h0 < p.hi ? 1u : 0u;
    const u64 hi = h0 + cy, c3 = hi < h0 ? 1u : 0u;
    const u64 r = gl_reduce128(lo, hi);
    return (c2 | c3) ? gl_sub(r, 1ull << 32) : r;
#endif
}

// Signed small integer to field (field.rs:32-34).
GL_HD u64 gl_from_i64(long long v) {
    if (v >= 0) return gl_canon((u64)v);
    u64 m = (u64)(-(v + 1)) + 1;
    return gl_canon(GL_P - m % GL_P);
}

GL_HD u64 gl_pow(u64 b, u64 e) {
    u64 acc = 1;
    while (e) {
        if (e & 1) acc = gl_mul(acc, b);
        b = gl_mul(b, b);
        e >>= 1;
    }
    return acc;
}
GL_HD u64 gl_sqn(u64 a, int n) {
    for (int i = 0; i < n; i++) a = gl_mul(a, a);
    return a;
}
// a^(p-2) by an addition chain: p - 2 = (2^32 - 2) 2^32 + (2^32 - 1); 64 squarings, 10 multiplies.
// The inverse is unique, so this is the word Fp::inv (field.rs:80-83) returns.
GL_HD u64 gl_inv(u64 a) {
    u64 a2 = gl_mul(gl_sqn(a, 1), a);         // a^(2^2 - 1)
    u64 a4 = gl_mul(gl_sqn(a2, 2), a2);       // a^(2^4 - 1)
    u64 a8 = gl_mul(gl_sqn(a4, 4), a4);
    u64 a16 = gl_mul(gl_sqn(a8, 8), a8);
    u64 a24 = gl_mul(gl_sqn(a16, 8), a8);
    u64 a28 = gl_mul(gl_sqn(a24, 4), a4);
    u64 a30 = gl_mul(gl_sqn(a28, 2), a2);
    u64 a31 = gl_mul(gl_sqn(a30, 1), a);      // a^(2^31 - 1)
    u64 b = gl_sqn(a31, 1);                   // a^(2^32 - 2)
    u64 a32 = gl_mul(b, a);                   // a^(2^32 - 1)
    return gl_mul(gl_sqn(b, 32), a32);
}

// canonical product through the carry-chain multiply (device) / the plain one (host)
GL_HD u64 gl_mul_fast(u64 a, u64 b) { return gl_canon_fast(gl_mul_lazy(a, b)); }

GL_HD fp2 f2(u64 a, u64 b) {
    fp2 r;
    r.c0 = a;
    r.c1 = b;
    return r;
}
GL_HD fp2 f2_add(fp2 a, fp2 b) { return f2(gl_add(a.c0, b.c0), gl_add(a.c1, b.c1)); }
GL_HD fp2 f2_sub(fp2 a, fp2 b) { return f2(gl_sub(a.c0, b.c0), gl_sub(a.c1, b.c1)); }
GL_HD fp2 f2_neg(fp2 a) { return f2(gl_neg(a.c0), gl_neg(a.c1)); }
GL_HD fp2 f2_mul_base(fp2 a, u64 b) { return f2(gl_mul(a.c0, b), gl_mul(a.c1, b)); }
// (a0 + a1 u)(b0 + b1 u) with u^2 = 7 (field.rs:163-169)
GL_HD fp2 f2_mul(fp2 a, fp2 b) {
#ifdef GL_DEVICE_CHAINS
    const u64 a17 = gl_sub_lazy(gl_add_lazy(a.c1 << 3, (a.c1 >> 61) * GL_EPS), a.c1);  // 7 a1 = 8 a1 - a1, a lazy word (the products take any word)
#else
    const u64 a17 = gl_sub(gl_reduce128(a.c1 << 3, a.c1 >> 61), a.c1);  // 7 a1 = 8 a1 - a1
#endif
    return f2(gl_mul_add2(a.c0, b.c0, a17, b.c1), gl_mul_add2(a.c0, b.c1, a.c1, b.c0));
}
GL_HD bool f2_is_zero(fp2 a) { return (a.c0 | a.c1) == 0; }
// conj(a) / (a0^2 - 7 a1^2) (field.rs:180-185)
GL_HD fp2 f2_inv(fp2 a) {
    u64 norm = gl_sub(gl_mul(a.c0, a.c0), gl_mul(gl_mul(a.c1, a.c1), 7));
    u64 ni = gl_inv(norm);
    return f2(gl_mul(a.c0, ni), gl_mul(gl_neg(a.c1), ni));
}

GL_HD u32 gl_brev(u32 x, int bits) {
#ifdef __CUDA_ARCH__
    return bits ? (__brev(x) >> (32 - bits)) : 0;
#else
    u32 r = 0;
    for (int i = 0; i < bits; i++) r = (r << 1) | ((x >> i) & 1);
    return r;
#endif
}
