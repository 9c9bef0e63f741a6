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
#include <vector>

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

// a b where either may lie in the base field (imaginary word zero): one or two base multiplications instead of
// the extension product's four.  Witness planes and public shape tables are base-valued until the first fold
// (slot_ir.rs:160-177), which is half of a sumcheck's work; within a warp the test goes the same way for every lane.
GL_HD fp2 mul_mixed(fp2 a, fp2 b) {
    if (a.c1 == 0) return b.c1 == 0 ? f2(gl_mul(a.c0, b.c0), 0) : f2_mul_base(b, a.c0);
    if (b.c1 == 0) return f2_mul_base(a, b.c0);
    return f2_mul(a, b);
}

GL_HD fp2 coef_mul(u32 ci, const fp2* cf, fp2 x) {
    if (ci == IR_ONE) return x;
    if (ci == IR_NEG_ONE) return f2_neg(x);
    if (ci == IR_ZERO) return f2(0, 0);
    return mul_mixed(cf[ci], x);
}

GL_HD fp2 factor_value(u32 f, const fp2* tv, const fp2* nv) { return (f & IR_NODE) ? nv[f & ~IR_NODE] : tv[f]; }

// coef * prod(factors) of one subterm or term; `pc` moves past it
GL_HD fp2 product(const u32* w, u32& pc, const fp2* cf, const fp2* tv, const fp2* nv) {
    const u32 ci = w[pc++], nf = w[pc++];
    if (nf == 0) return coef_value(ci, cf);
    fp2 p = factor_value(w[pc++], tv, nv);
    for (u32 i = 1; i < nf; i++) p = mul_mixed(p, factor_value(w[pc++], tv, nv));
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

// ---------------------------------------------------------------------------------------------
// The evaluation plan: the same graph regrouped for the kernels.  Every node becomes a sum of UNITS
// (coef * prod(factors); an affine term is a unit with one table factor, its constant a unit with none),
// the top-level terms become the units of one more node (id n_nodes) whose value is the polynomial, and
// the nodes are ordered by LEVEL (a node's level is one more than the highest level it refers to), so
// that all units of a level are independent: a thread walks them in order, a warp takes one unit per lane.
//
//   pw[0] levels  pw[1] nodes (with the final one)  pw[2] units
//   pw[3..7] offsets of: level -> first node (levels + 1), node -> id (nodes), node -> first unit (nodes + 1),
//                        unit -> offset of its record (units), the unit records [coef] [nf] nf x [factor]
//   pw[8] total words
// A level never holds more than PLAN_LEVEL_UNITS units (wider levels are cut: their nodes are independent).
// ---------------------------------------------------------------------------------------------
constexpr u32 PLAN_HEAD = 9, PLAN_LEVEL_UNITS = 256, PLAN_MAX_WORDS = 8192;

// returns 0 and fills `pw`, or a non-zero reason (a node wider than a level, a plan beyond PLAN_MAX_WORDS)
inline int build_plan(const Shape& s, const u32* w, std::vector<u32>& pw) {
    struct Node { u32 id, level; std::vector<std::vector<u32>> units; };
    std::vector<Node> nodes(s.n_nodes + 1);
    std::vector<u32> level(s.n_nodes + 1, 0);
    u32 pc = 0;
    auto read_product = [&](Node& nd) {
        const u32 ci = w[pc++], nf = w[pc++];
        std::vector<u32> u{ci, nf};
        for (u32 i = 0; i < nf; i++) {
            const u32 f = w[pc++];
            u.push_back(f);
            if (f & IR_NODE) nd.level = nd.level > level[f & ~IR_NODE] + 1 ? nd.level : level[f & ~IR_NODE] + 1;
        }
        nd.units.push_back(u);
    };
    for (u32 n = 0; n <= s.n_nodes; n++) {
        Node& nd = nodes[n];
        nd.id = n;
        nd.level = 1;
        if (n == s.n_nodes) {
            for (u32 t = 0; t < s.n_terms; t++) read_product(nd);
            for (u32 m = 0; m < s.n_nodes; m++) nd.level = nd.level > level[m] + 1 ? nd.level : level[m] + 1;  // the last level, alone
        } else {
            const u32 head = w[pc++], cnt = head >> 8;
            if ((head & 0xFFu) == IR_AFFINE) {
                const u32 kc = w[pc++];
                if (kc != IR_ZERO) nd.units.push_back({kc, 0u});
                for (u32 i = 0; i < cnt; i++, pc += 2) nd.units.push_back({w[pc], 1u, w[pc + 1]});
            } else {
                for (u32 i = 0; i < cnt; i++) read_product(nd);
            }
        }
        if (nd.units.size() > PLAN_LEVEL_UNITS) return 1;
        level[n] = nd.level;
    }
    // order by level (stable in the id), cutting levels that are too wide
    std::vector<u32> order;
    std::vector<u32> lvl_start{0};
    u32 maxl = 0;
    for (auto& nd : nodes) maxl = nd.level > maxl ? nd.level : maxl;
    for (u32 l = 1; l <= maxl; l++) {
        u32 in_level = 0;
        bool any = false;
        for (auto& nd : nodes) {
            if (nd.level != l) continue;
            if (any && in_level + nd.units.size() > PLAN_LEVEL_UNITS) {
                lvl_start.push_back((u32)order.size());
                in_level = 0;
            }
            order.push_back(nd.id);
            in_level += (u32)nd.units.size();
            any = true;
        }
        if (any) lvl_start.push_back((u32)order.size());
    }
    const u32 L = (u32)lvl_start.size() - 1, NN = (u32)order.size();
    std::vector<u32> nus{0}, uoff, uw;
    for (u32 k = 0; k < NN; k++) {
        for (auto& u : nodes[order[k]].units) {
            uoff.push_back((u32)uw.size());
            uw.insert(uw.end(), u.begin(), u.end());
        }
        nus.push_back((u32)uoff.size());
    }
    pw.assign(PLAN_HEAD, 0);
    pw[0] = L; pw[1] = NN; pw[2] = (u32)uoff.size();
    pw[3] = (u32)pw.size(); pw.insert(pw.end(), lvl_start.begin(), lvl_start.end());
    pw[4] = (u32)pw.size(); pw.insert(pw.end(), order.begin(), order.end());
    pw[5] = (u32)pw.size(); pw.insert(pw.end(), nus.begin(), nus.end());
    pw[6] = (u32)pw.size(); pw.insert(pw.end(), uoff.begin(), uoff.end());
    pw[7] = (u32)pw.size(); pw.insert(pw.end(), uw.begin(), uw.end());
    pw[8] = (u32)pw.size();
    return pw.size() > PLAN_MAX_WORDS ? 2 : 0;
}

// one thread walks the whole plan; nv holds n_nodes + 1 values, the last one is the polynomial
GL_HD fp2 plan_eval(const u32* pw, const fp2* cf, const fp2* tv, fp2* nv) {
    const u32 NN = pw[1];
    const u32 *nid = pw + pw[4], *nus = pw + pw[5], *uoff = pw + pw[6], *uw = pw + pw[7];
    fp2 acc = f2(0, 0);
    for (u32 n = 0; n < NN; n++) {
        acc = f2(0, 0);
        for (u32 u = nus[n]; u < nus[n + 1]; u++) {
            u32 pc = uoff[u];
            acc = f2_add(acc, product(uw, pc, cf, tv, nv));
        }
        nv[nid[n]] = acc;
    }
    return acc;  // the final node is last in the order
}

// The same plan by `lanes` cooperating workers (a warp on the device; the host emulation runs the lanes of a
// phase one after another).  Phase A of a level: lane takes units u0 + lane, + lanes, ... into ub; phase B: lane takes
// nodes and sums their units.  The caller separates the phases with a barrier over the lanes.
GL_HD void plan_level_units(const u32* pw, u32 l, const fp2* cf, const fp2* tv, const fp2* nv, fp2* ub, u32 lane, u32 lanes) {
    const u32 *lvl = pw + pw[3], *nus = pw + pw[5], *uoff = pw + pw[6], *uw = pw + pw[7];
    const u32 u0 = nus[lvl[l]], u1 = nus[lvl[l + 1]];
    for (u32 u = u0 + lane; u < u1; u += lanes) {
        u32 pc = uoff[u];
        ub[u - u0] = product(uw, pc, cf, tv, nv);
    }
}
GL_HD void plan_level_nodes(const u32* pw, u32 l, const fp2* ub, fp2* nv, u32 lane, u32 lanes) {
    const u32 *lvl = pw + pw[3], *nid = pw + pw[4], *nus = pw + pw[5];
    const u32 n0 = lvl[l], n1 = lvl[l + 1], u0 = nus[n0];
    for (u32 n = n0 + lane; n < n1; n += lanes) {
        fp2 acc = f2(0, 0);
        for (u32 u = nus[n]; u < nus[n + 1]; u++) acc = f2_add(acc, ub[u - u0]);
        nv[nid[n]] = acc;
    }
}

}  // namespace ir
