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
// Called, not inlined, on the device: the evaluators' loops are unrolled over the points, and a copy of the four
// multiplication forms at every site makes kernels that wait on instruction fetch (measured: a quarter of all stall
// cycles of the thread pair form).
#ifdef __CUDACC__
#define IR_CALL static __host__ __device__ __noinline__
#else
#define IR_CALL inline
#endif
IR_CALL fp2 mul_mixed(fp2 a, fp2 b) {
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

// The SIGNATURE of a well-formed stream: FNV-1a over (n_tables, n_nodes, n_terms) and the stream's words with every
// coefficient word replaced by the coefficient's class (the special words as they are; a general coefficient by whether
// its value lies in the base field), so that a graph is recognised whatever its challenges are.  The generated kernels
// (slot_gen.cuh) are keyed by it and read their coefficients by OCCURRENCE: `by_occurrence` receives the value of the
// j-th coefficient word of the stream.
constexpr u32 IR_CLASS_BASE = 0xFFFFFFF0u, IR_CLASS_EXT = 0xFFFFFFF1u;
inline u64 signature(const Shape& s, const u32* w, const fp2* cf, std::vector<fp2>* by_occurrence) {
    u64 h = 0xCBF29CE484222325ull;
    auto mix = [&](u32 word) {
        for (int b = 0; b < 4; b++) h = (h ^ ((word >> (8 * b)) & 0xFFu)) * 0x100000001B3ull;
    };
    auto coef = [&](u32 ci) {
        const fp2 v = coef_value(ci, cf);
        if (by_occurrence) by_occurrence->push_back(v);
        mix((ci == IR_ONE || ci == IR_NEG_ONE || ci == IR_ZERO) ? ci : (v.c1 == 0 ? IR_CLASS_BASE : IR_CLASS_EXT));
    };
    mix(s.n_tables); mix(s.n_nodes); mix(s.n_terms);
    u32 pc = 0;
    auto product = [&]() {
        coef(w[pc++]);
        const u32 nf = w[pc++];
        mix(nf);
        for (u32 i = 0; i < nf; i++) mix(w[pc++]);
    };
    for (u32 n = 0; n < s.n_nodes; n++) {
        const u32 head = w[pc++], cnt = head >> 8;
        mix(head);
        if ((head & 0xFFu) == IR_AFFINE) {
            coef(w[pc++]);
            for (u32 i = 0; i < cnt; i++) { coef(w[pc++]); mix(w[pc++]); }
        } else {
            for (u32 i = 0; i < cnt; i++) product();
        }
    }
    for (u32 t = 0; t < s.n_terms; t++) product();
    return h;
}

// ---------------------------------------------------------------------------------------------
// The evaluation plan: the same graph regrouped for the kernels.  Every node becomes a sum of UNITS
// (coef * prod(factors); an affine term is a unit with one table factor, its constant a unit with none),
// the top-level terms become the units of one more node (id n_nodes) whose value is the polynomial.
// Node order: the affine nodes first, then the others by LEVEL (one more than the highest level a node
// refers to), so that a single pass over the order is a valid evaluation and all units of a level are
// independent.
//
//   pw[0]  sum levels          pw[1]  nodes (with the final one)      pw[2]  units
//   pw[3]  -> level bounds over the node order, levels + 1 entries, first = pw[9] (the non-affine nodes,
//             each level at most `level_cap` units: wider levels are cut, their nodes are independent)
//   pw[4]  -> node id per position        pw[5]  -> first unit per position (nodes + 1)
//   pw[6]  -> record offset per unit      pw[7]  -> the unit records [coef] [nf] nf x [factor]
//   pw[8]  total words                    pw[9]  affine nodes (positions 0 .. pw[9])
//   pw[10] -> bounds of the affine groups (at most PLAN_AFFINE_GROUP units each), pw[11] + 1 entries
//   pw[13] -> the LIVE tables (read directly by a non-affine node or a term), pw[14] of them
//   pw[16] the degree the graph ATTAINS along one variable (every table counts 1; slot_ir.rs:380-413): the round
//             polynomial is evaluated at 0 .. min(declared, attained) only, the points above follow by exact
//             extrapolation (gpu/metal.rs:2516-2548 does the same)
//   pw[12] -> a second copy of the non-affine nodes' unit records with COMPACT factor words: live table j -> j,
//             node -> pw[14] + its position in the node order (record offsets relative to the first such unit),
//             pw[15] -> their record offsets; the thread pair form keeps only these values in local memory
//
// Along a sumcheck round's variable every table is affine in the evaluation point d, T(i) + d (T(i+half) - T(i)),
// hence so is every affine node: value at d = 0 and difference are computed once per pair and the other points
// follow by additions; only the remaining ("sum") nodes are evaluated at every point.
// ---------------------------------------------------------------------------------------------
constexpr u32 PLAN_HEAD = 17, PLAN_UNIT_BUF = 256, PLAN_AFFINE_GROUP = PLAN_UNIT_BUF / 2, PLAN_MAX_WORDS = 8192;

// the degree a well-formed stream attains along one variable
inline u32 attained_degree(const Shape& s, const u32* w) {
    std::vector<u32> deg(s.n_nodes, 0);
    u32 pc = 0, top = 0;
    auto prod_deg = [&]() {
        const u32 nf = w[pc + 1];
        u32 d = 0;
        for (u32 i = 0; i < nf; i++) d += (w[pc + 2 + i] & IR_NODE) ? deg[w[pc + 2 + i] & ~IR_NODE] : 1u;
        pc += 2 + nf;
        return d;
    };
    for (u32 n = 0; n < s.n_nodes; n++) {
        const u32 head = w[pc++], cnt = head >> 8;
        u32 d = 0;
        if ((head & 0xFFu) == IR_AFFINE) {
            d = cnt ? 1u : 0u;
            pc += 1 + 2 * cnt;
        } else {
            for (u32 i = 0; i < cnt; i++) { const u32 x = prod_deg(); d = x > d ? x : d; }
        }
        deg[n] = d;
    }
    for (u32 t = 0; t < s.n_terms; t++) { const u32 x = prod_deg(); top = x > top ? x : top; }
    return top;
}

// degree: the slot's declared degree; the plan evaluates min(declared, attained) + 1 points, and a sum level holds at
// most PLAN_UNIT_BUF / points units (the pair form runs a level's units at every point at once).
// Returns 0 and fills `pw`, or a non-zero reason (a node wider than a level, a plan beyond PLAN_MAX_WORDS).
inline int build_plan(const Shape& s, const u32* w, u32 degree, std::vector<u32>& pw) {
    struct Node { u32 id, level; bool affine = false; std::vector<std::vector<u32>> units; };
    std::vector<Node> nodes(s.n_nodes + 1);
    std::vector<u32> level(s.n_nodes + 1, 0);
    const u32 attained = attained_degree(s, w), de = attained < degree ? attained : degree;
    const u32 level_cap = PLAN_UNIT_BUF / (de + 1);
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
                nd.affine = true;
                const u32 kc = w[pc++];
                if (kc != IR_ZERO) nd.units.push_back({kc, 0u});
                for (u32 i = 0; i < cnt; i++, pc += 2) nd.units.push_back({w[pc], 1u, w[pc + 1]});
            } else {
                for (u32 i = 0; i < cnt; i++) read_product(nd);
            }
        }
        if (nd.units.size() > (nd.affine ? PLAN_AFFINE_GROUP : level_cap)) return 1;
        level[n] = nd.level;
    }
    std::vector<u32> order, agrp{0}, lvl;
    u32 in_group = 0;
    for (auto& nd : nodes) {  // affine nodes, grouped
        if (!nd.affine) continue;
        if (in_group + nd.units.size() > PLAN_AFFINE_GROUP) { agrp.push_back((u32)order.size()); in_group = 0; }
        order.push_back(nd.id);
        in_group += (u32)nd.units.size();
    }
    const u32 NA = (u32)order.size();
    if (agrp.back() != NA) agrp.push_back(NA);
    lvl.push_back(NA);
    u32 maxl = 0;
    for (auto& nd : nodes) maxl = nd.level > maxl ? nd.level : maxl;
    for (u32 l = 1; l <= maxl; l++) {  // the others by level (stable in the id), cutting levels that are too wide
        u32 in_level = 0;
        bool any = false;
        for (auto& nd : nodes) {
            if (nd.affine || nd.level != l) continue;
            if (any && in_level + nd.units.size() > level_cap) { lvl.push_back((u32)order.size()); in_level = 0; }
            order.push_back(nd.id);
            in_level += (u32)nd.units.size();
            any = true;
        }
        if (any) lvl.push_back((u32)order.size());
    }
    const u32 NN = (u32)order.size();
    std::vector<u32> nus{0}, uoff, uw, live;
    std::vector<bool> is_live(s.n_tables, false);
    for (u32 k = 0; k < NN; k++) {
        const Node& nd = nodes[order[k]];
        for (auto& u : nd.units) {
            uoff.push_back((u32)uw.size());
            uw.insert(uw.end(), u.begin(), u.end());
            if (!nd.affine)
                for (size_t f = 2; f < u.size(); f++)
                    if (!(u[f] & IR_NODE)) is_live[u[f]] = true;
        }
        nus.push_back((u32)uoff.size());
    }
    for (u32 t = 0; t < s.n_tables; t++)
        if (is_live[t]) live.push_back(t);
    pw.assign(PLAN_HEAD, 0);
    pw[16] = de;
    pw[0] = (u32)lvl.size() - 1; pw[1] = NN; pw[2] = (u32)uoff.size(); pw[9] = NA; pw[11] = (u32)agrp.size() - 1; pw[14] = (u32)live.size();
    pw[3] = (u32)pw.size(); pw.insert(pw.end(), lvl.begin(), lvl.end());
    pw[4] = (u32)pw.size(); pw.insert(pw.end(), order.begin(), order.end());
    pw[5] = (u32)pw.size(); pw.insert(pw.end(), nus.begin(), nus.end());
    pw[6] = (u32)pw.size(); pw.insert(pw.end(), uoff.begin(), uoff.end());
    pw[7] = (u32)pw.size(); pw.insert(pw.end(), uw.begin(), uw.end());
    pw[10] = (u32)pw.size(); pw.insert(pw.end(), agrp.begin(), agrp.end());
    pw[13] = (u32)pw.size(); pw.insert(pw.end(), live.begin(), live.end());
    {   // compact records of the non-affine nodes' units
        std::vector<u32> slot_of_table(s.n_tables, 0), pos_of_node(s.n_nodes + 1, 0), cw, coff;
        for (u32 j = 0; j < live.size(); j++) slot_of_table[live[j]] = j;
        for (u32 k = 0; k < NN; k++) pos_of_node[order[k]] = k;
        for (u32 k = NA; k < NN; k++)
            for (auto& u : nodes[order[k]].units) {
                coff.push_back((u32)cw.size());
                cw.push_back(u[0]);
                cw.push_back(u[1]);
                for (size_t f = 2; f < u.size(); f++)
                    cw.push_back((u[f] & IR_NODE) ? (u32)live.size() + pos_of_node[u[f] & ~IR_NODE] : slot_of_table[u[f]]);
            }
        pw[12] = (u32)pw.size(); pw.insert(pw.end(), cw.begin(), cw.end());
        pw[15] = (u32)pw.size(); pw.insert(pw.end(), coff.begin(), coff.end());
    }
    pw[8] = (u32)pw.size();
    return pw.size() > PLAN_MAX_WORDS ? 2 : 0;
}

// ---- thread form: one worker walks the whole plan at ONE point; nv holds n_nodes + 1 values ----
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

// ---- thread pair form: one worker, one pair, every point, with a compact value array:
// V[j] live table j, V[n_live + k] the node at position k; D[j], D[n_live + k] the differences of the live tables and
// of the affine nodes (positions below pw[9]).  The affine nodes read their tables through `table(t, lo, dif)`. ----
template <class Table>
GL_HD void tpair_affine(const u32* pw, const fp2* cf, fp2* V, fp2* D, Table table) {
    const u32 *nus = pw + pw[5], *uoff = pw + pw[6], *uw = pw + pw[7];
    const u32 nl = pw[14], na = pw[9];
    for (u32 k = 0; k < na; k++) {
        fp2 v = f2(0, 0), d = f2(0, 0);
        for (u32 u = nus[k]; u < nus[k + 1]; u++) {
            const u32* r = uw + uoff[u];
            if (r[1] == 0) {
                v = f2_add(v, coef_value(r[0], cf));
            } else {
                fp2 lo, df;
                table(r[2], lo, df);
                v = f2_add(v, coef_mul(r[0], cf, lo));
                d = f2_add(d, coef_mul(r[0], cf, df));
            }
        }
        V[nl + k] = v;
        D[nl + k] = d;
    }
}
GL_HD void tpair_step(const u32* pw, fp2* V, const fp2* D) {
    for (u32 j = 0; j < pw[14] + pw[9]; j++) V[j] = f2_add(V[j], D[j]);
}
// the non-affine nodes at the current point; returns the polynomial's value
GL_HD fp2 tpair_sums(const u32* pw, const fp2* cf, fp2* V) {
    const u32 *nus = pw + pw[5], *cw = pw + pw[12], *coff = pw + pw[15];
    const u32 nl = pw[14], na = pw[9], nn = pw[1], u_base = nus[na];
    fp2 acc = f2(0, 0);
    for (u32 k = na; k < nn; k++) {
        acc = f2(0, 0);
        for (u32 u = nus[k]; u < nus[k + 1]; u++) {
            const u32* r = cw + coff[u - u_base];
            fp2 x;
            if (r[1] == 0) {
                x = coef_value(r[0], cf);
            } else {
                x = V[r[2]];
                for (u32 i = 1; i < r[1]; i++) x = mul_mixed(x, V[r[2 + i]]);
                x = coef_mul(r[0], cf, x);
            }
            acc = f2_add(acc, x);
        }
        V[nl + k] = acc;
    }
    return acc;
}

// The same, unit by unit with every point at once: a unit's record is decoded ONCE per pair, its affine-type factors
// (live tables, affine nodes) are stepped in registers, and the products of the points are independent chains.
// W[(k - na) * npw + p] holds the non-affine node at position k at point p (npw = points evaluated, at most
// TPAIR_POINTS); out receives the final node's values.  With skip_one the point 1 is left zero.
constexpr u32 TPAIR_POINTS = 6, TPAIR_SUM_NODES = 40, TPAIR_AFFINE_VALUES = 128;
GL_HD bool tpair_all_fits(const u32* pw) {
    return pw[16] + 1 <= TPAIR_POINTS && pw[1] - pw[9] <= TPAIR_SUM_NODES && pw[14] + pw[9] <= TPAIR_AFFINE_VALUES;
}
// NPW = points evaluated (pw[16] + 1), SKIP = the point 1 is not evaluated: compile-time, so that the unrolled point loops
// carry no tests.
template <u32 NPW, bool SKIP>
GL_HD void tpair_sums_all_t(const u32* pw, const fp2* cf, const fp2* V, const fp2* D, fp2* W, fp2* out) {
    const u32 *nus = pw + pw[5], *cw = pw + pw[12], *coff = pw + pw[15];
    const u32 nl = pw[14], na = pw[9], nn = pw[1], u_base = nus[na], naff = nl + na;
    fp2 acc[NPW];
    for (u32 k = na; k < nn; k++) {
#pragma unroll
        for (u32 p = 0; p < NPW; p++) acc[p] = f2(0, 0);
        for (u32 u = nus[k]; u < nus[k + 1]; u++) {
            const u32* r = cw + coff[u - u_base];
            const u32 ci = r[0], nf = r[1];
            fp2 x[NPW];
            if (nf == 0) {
                const fp2 c = coef_value(ci, cf);
#pragma unroll
                for (u32 p = 0; p < NPW; p++) x[p] = c;
            } else {
                // first factor with the coefficient folded in: coef (v + p d) = coef v + p (coef d) for an affine-type factor
                const u32 s0 = r[2];
                if (s0 < naff) {
                    fp2 v = coef_mul(ci, cf, V[s0]);
                    const fp2 d = coef_mul(ci, cf, D[s0]);
#pragma unroll
                    for (u32 p = 0; p < NPW; p++) {
                        x[p] = v;
                        if (p + 1 < NPW) v = f2_add(v, d);
                    }
                } else {
#pragma unroll
                    for (u32 p = 0; p < NPW; p++)
                        if (!(SKIP && p == 1)) x[p] = coef_mul(ci, cf, W[(s0 - naff) * NPW + p]);
                }
                for (u32 i = 1; i < nf; i++) {
                    const u32 si = r[2 + i];
                    if (si < naff) {
                        fp2 v = V[si];
                        const fp2 d = D[si];
#pragma unroll
                        for (u32 p = 0; p < NPW; p++) {
                            if (!(SKIP && p == 1)) x[p] = mul_mixed(x[p], v);
                            if (p + 1 < NPW) v = f2_add(v, d);
                        }
                    } else {
#pragma unroll
                        for (u32 p = 0; p < NPW; p++)
                            if (!(SKIP && p == 1)) x[p] = mul_mixed(x[p], W[(si - naff) * NPW + p]);
                    }
                }
            }
#pragma unroll
            for (u32 p = 0; p < NPW; p++)
                if (!(SKIP && p == 1)) acc[p] = f2_add(acc[p], x[p]);
        }
#pragma unroll
        for (u32 p = 0; p < NPW; p++) W[(k - na) * NPW + p] = (SKIP && p == 1) ? f2(0, 0) : acc[p];
    }
#pragma unroll
    for (u32 p = 0; p < TPAIR_POINTS; p++) out[p] = f2(0, 0);
#pragma unroll
    for (u32 p = 0; p < NPW; p++)
        if (!(SKIP && p == 1)) out[p] = acc[p];
}

// host-side dispatch for the emulation (the kernels are instantiated per point count)
inline void tpair_sums_all(const u32* pw, const fp2* cf, const fp2* V, const fp2* D, fp2* W, bool skip_one, fp2* out) {
    const u32 npw = pw[16] + 1;
#define IR_TP(N) case N: if (skip_one) tpair_sums_all_t<N, true>(pw, cf, V, D, W, out); else tpair_sums_all_t<N, false>(pw, cf, V, D, W, out); break;
    switch (npw) { IR_TP(1) IR_TP(2) IR_TP(3) IR_TP(4) IR_TP(5) IR_TP(6) }
#undef IR_TP
}

// ---- pair form: `lanes` cooperating workers (a warp; the host emulation runs the lanes of a phase one after
// another) evaluate ONE pair at every point.  Values live in V[id * np + point] (id = table, or n_tables + node id),
// differences in DV[id], products of the running phase in UB (PLAN_UNIT_BUF entries).  The caller fills V[t * np]
// and DV[t] for every table and separates the phases with a barrier over the lanes. ----
struct Pair {
    const u32* pw;
    const fp2* cf;
    fp2 *V, *DV, *UB;
    u32 n_tables, np;   // np = declared degree + 1
    u32 npe;            // points evaluated: np, or np - 1 when the point 1 comes from the running claim
    GL_HD u32 point(u32 pi) const { return npe == np || pi == 0 ? pi : pi + 1; }
};

// affine group g, phase 1: the units' products at point 0 (UB[j]) and along the difference (UB[half + j])
GL_HD void pair_affine_units(const Pair& a, u32 g, u32 lane, u32 lanes) {
    const u32 *grp = a.pw + a.pw[10], *nus = a.pw + a.pw[5], *uoff = a.pw + a.pw[6], *uw = a.pw + a.pw[7];
    const u32 u0 = nus[grp[g]], u1 = nus[grp[g + 1]];
    for (u32 u = u0 + lane; u < u1; u += lanes) {
        const u32* r = uw + uoff[u];
        if (r[1] == 0) {
            a.UB[u - u0] = coef_value(r[0], a.cf);
            a.UB[PLAN_AFFINE_GROUP + u - u0] = f2(0, 0);
        } else {
            a.UB[u - u0] = coef_mul(r[0], a.cf, a.V[r[2] * a.np]);
            a.UB[PLAN_AFFINE_GROUP + u - u0] = coef_mul(r[0], a.cf, a.DV[r[2]]);
        }
    }
}
// phase 2: the group's nodes sum their units
GL_HD void pair_affine_nodes(const Pair& a, u32 g, u32 lane, u32 lanes) {
    const u32 *grp = a.pw + a.pw[10], *nid = a.pw + a.pw[4], *nus = a.pw + a.pw[5];
    const u32 k0 = grp[g], k1 = grp[g + 1], u0 = nus[k0];
    for (u32 k = k0 + lane; k < k1; k += lanes) {
        fp2 v = f2(0, 0), d = f2(0, 0);
        for (u32 u = nus[k]; u < nus[k + 1]; u++) {
            v = f2_add(v, a.UB[u - u0]);
            d = f2_add(d, a.UB[PLAN_AFFINE_GROUP + u - u0]);
        }
        const u32 id = a.n_tables + nid[k];
        a.V[id * a.np] = v;
        a.DV[id] = d;
    }
}
// live tables and affine nodes at the points 1 .. np - 1, by additions
GL_HD void pair_step(const Pair& a, u32 lane, u32 lanes) {
    const u32 *live = a.pw + a.pw[13], *nid = a.pw + a.pw[4];
    const u32 nl = a.pw[14], na = a.pw[9];
    for (u32 j = lane; j < nl + na; j += lanes) {
        const u32 id = j < nl ? live[j] : a.n_tables + nid[j - nl];
        fp2 v = a.V[id * a.np];
        const fp2 d = a.DV[id];
        for (u32 p = 1; p < a.np; p++) { v = f2_add(v, d); a.V[id * a.np + p] = v; }
    }
}
GL_HD fp2 pair_product(const Pair& a, const u32* r, u32 p) {
    const u32 nf = r[1];
    if (nf == 0) return coef_value(r[0], a.cf);
    auto val = [&](u32 f) { return a.V[((f & IR_NODE) ? a.n_tables + (f & ~IR_NODE) : f) * a.np + p]; };
    fp2 x = val(r[2]);
    for (u32 i = 1; i < nf; i++) x = mul_mixed(x, val(r[2 + i]));
    return coef_mul(r[0], a.cf, x);
}
// sum level l, phase 1: every (unit, evaluated point) product
GL_HD void pair_level_units(const Pair& a, u32 l, u32 lane, u32 lanes) {
    const u32 *lvl = a.pw + a.pw[3], *nus = a.pw + a.pw[5], *uoff = a.pw + a.pw[6], *uw = a.pw + a.pw[7];
    const u32 u0 = nus[lvl[l]], u1 = nus[lvl[l + 1]];
    for (u32 x = lane; x < (u1 - u0) * a.npe; x += lanes) {
        const u32 u = x / a.npe, pi = x - u * a.npe;
        a.UB[x] = pair_product(a, uw + uoff[u0 + u], a.point(pi));
    }
}
// phase 2: every (node, evaluated point) sum
GL_HD void pair_level_nodes(const Pair& a, u32 l, u32 lane, u32 lanes) {
    const u32 *lvl = a.pw + a.pw[3], *nid = a.pw + a.pw[4], *nus = a.pw + a.pw[5];
    const u32 k0 = lvl[l], k1 = lvl[l + 1], u0 = nus[k0];
    for (u32 x = lane; x < (k1 - k0) * a.npe; x += lanes) {
        const u32 k = k0 + x / a.npe, pi = x % a.npe;
        fp2 v = f2(0, 0);
        for (u32 u = nus[k]; u < nus[k + 1]; u++) v = f2_add(v, a.UB[(u - u0) * a.npe + pi]);
        a.V[(a.n_tables + nid[k]) * a.np + a.point(pi)] = v;
    }
}
// Fp2 entries of one worker group's areas: V, DV, UB
GL_HD u32 pair_area(u32 n_tables, u32 n_nodes_with_final, u32 np) { return (n_tables + n_nodes_with_final) * (np + 1) + PLAN_UNIT_BUF; }

}  // namespace ir
