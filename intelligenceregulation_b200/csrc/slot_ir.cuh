// A slot polynomial given as data: the expression graph of private_block/slot_ir.rs:57-345 flattened
// into 32-bit words, and its evaluation at one cube point (the interpreter of slot_ir.rs:352-377).
//
//   polynomial = sum over terms of    coef * prod(factors)
//   factor     = a table's value at the point, or a node's value
//   node       = affine:  konst + sum_i coef_i * table_i
//                sum:     sum over subterms of coef * prod(factors)      (nodes only refer back)
//
// Word stream: the node records in order, then the term records.
//   affine node   [IR_AFFINE | count << 8] [konst coef] count x ([coef] [table])
//   sum node      [IR_SUM    | count << 8] count x ( [coef] [nf] nf x [factor] )
//   term          [coef] [nf] nf x [factor]          (wrapper tables first, then the inner factors)
//   factor        table id, or IR_NODE | node id
//   coef          index into the Fp2 coefficient array, or IR_ONE / IR_NEG_ONE / IR_ZERO
//
// Field arithmetic is exact and results are canonical words, so the order of the additions and
// multiplications is free: any evaluator of the same graph returns the reference's words.
#pragma once
#include <cstddef>

#include "gl_field.cuh"

namespace ir {

constexpr u32 IR_AFFINE = 0, IR_SUM = 1;
constexpr u32 IR_NODE = 0x80000000u;
constexpr u32 IR_ONE = 0xFFFFFFFFu, IR_NEG_ONE = 0xFFFFFFFEu, IR_ZERO = 0xFFFFFFFDu;
constexpr u32 MAX_TABLES = 64, MAX_NODES = 128, MAX_WORDS = 4096, MAX_COEFS = 512;

struct Shape {
    u32 n_tables, n_nodes, n_terms, n_coefs, n_words;
};

GL_HD fp2 coef_value(u32 ci, const fp2* cf) {
    if (ci == IR_ONE) return f2(1, 0);
    if (ci == IR_NEG_ONE) return f2(GL_P - 1, 0);
    if (ci == IR_ZERO) return f2(0, 0);
    return cf[ci];
}

// coef * x; a base-field coefficient (imaginary word zero) costs two multiplications instead of five
GL_HD fp2 coef_mul(u32 ci, const fp2* cf, fp2 x) {
    if (ci == IR_ONE) return x;
    if (ci == IR_NEG_ONE) return f2_neg(x);
    if (ci == IR_ZERO) return f2(0, 0);
    const fp2 c = cf[ci];
    return c.c1 == 0 ? f2_mul_base(x, c.c0) : f2_mul(c, x);
}

GL_HD fp2 factor_value(u32 f, const fp2* tv, const fp2* nv) { return (f & IR_NODE) ? nv[f & ~IR_NODE] : tv[f]; }

// coef * prod(factors) of one subterm or term; `pc` moves past it
GL_HD fp2 product(const u32* w, u32& pc, const fp2* cf, const fp2* tv, const fp2* nv) {
    const u32 ci = w[pc++], nf = w[pc++];
    if (nf == 0) return coef_value(ci, cf);
    fp2 p = factor_value(w[pc++], tv, nv);
    for (u32 i = 1; i < nf; i++) p = f2_mul(p, factor_value(w[pc++], tv, nv));
    return coef_mul(ci, cf, p);
}

// the polynomial at one point: tv = the point's table values, nv = scratch for the node values
GL_HD fp2 eval(const Shape& s, const u32* w, const fp2* cf, const fp2* tv, fp2* nv) {
    u32 pc = 0;
    for (u32 n = 0; n < s.n_nodes; n++) {
        const u32 head = w[pc++], cnt = head >> 8;
        fp2 acc;
        if ((head & 0xFFu) == IR_AFFINE) {
            acc = coef_value(w[pc++], cf);
            for (u32 i = 0; i < cnt; i++) {
                const u32 ci = w[pc++], t = w[pc++];
                acc = f2_add(acc, coef_mul(ci, cf, tv[t]));
            }
        } else {
            acc = f2(0, 0);
            for (u32 i = 0; i < cnt; i++) acc = f2_add(acc, product(w, pc, cf, tv, nv));
        }
        nv[n] = acc;
    }
    fp2 total = f2(0, 0);
    for (u32 t = 0; t < s.n_terms; t++) total = f2_add(total, product(w, pc, cf, tv, nv));
    return total;
}

// Host-side check of a word stream before it reaches a kernel: every id in range, nodes refer back only,
// the stream ends exactly at n_words (the invariant of slot_ir.rs:445-489).  Returns 0 when well formed.
inline int validate(const Shape& s, const u32* w) {
    if (s.n_tables == 0 || s.n_tables > MAX_TABLES || s.n_nodes > MAX_NODES || s.n_words > MAX_WORDS || s.n_coefs > MAX_COEFS) return 1;
    u32 pc = 0;
    auto coef_ok = [&](u32 ci) { return ci == IR_ONE || ci == IR_NEG_ONE || ci == IR_ZERO || ci < s.n_coefs; };
    auto prod_ok = [&](u32 upto) {
        if (pc + 2 > s.n_words) return false;
        const u32 ci = w[pc++], nf = w[pc++];
        if (!coef_ok(ci) || nf > 64 || pc + nf > s.n_words) return false;
        for (u32 i = 0; i < nf; i++) {
            const u32 f = w[pc++];
            if (f & IR_NODE) { if ((f & ~IR_NODE) >= upto) return false; }
            else if (f >= s.n_tables) return false;
        }
        return true;
    };
    for (u32 n = 0; n < s.n_nodes; n++) {
        if (pc >= s.n_words) return 2;
        const u32 head = w[pc++], cnt = head >> 8, kind = head & 0xFFu;
        if (kind == IR_AFFINE) {
            if (pc + 1 + 2 * (size_t)cnt > s.n_words || !coef_ok(w[pc])) return 3;
            pc++;
            for (u32 i = 0; i < cnt; i++) {
                if (!coef_ok(w[pc]) || w[pc + 1] >= s.n_tables) return 4;
                pc += 2;
            }
        } else if (kind == IR_SUM) {
            for (u32 i = 0; i < cnt; i++)
                if (!prod_ok(n)) return 5;
        } else {
            return 6;
        }
    }
    for (u32 t = 0; t < s.n_terms; t++)
        if (!prod_ok(s.n_nodes)) return 7;
    return pc == s.n_words ? 0 : 8;
}

}  // namespace ir
