// Runs the product's slot-polynomial interpreter and its program check (csrc/slot_ir.cuh) on the host,
// so that the CPU test suite compares them with the oracle without a device.
#include "../../intelligenceregulation_b200/csrc/slot_ir.cuh"

extern "C" int emul_ir_validate(const u32* words, u32 n_words, u32 n_tables, u32 n_nodes, u32 n_terms, u32 n_coefs) {
    ir::Shape s{n_tables, n_nodes, n_terms, n_coefs, n_words};
    return ir::validate(s, words);
}

extern "C" void emul_ir_eval(const u32* words, u32 n_words, u32 n_tables, u32 n_nodes, u32 n_terms, const u64* coefs, u32 n_coefs,
                             const u64* values, u64* out) {
    ir::Shape s{n_tables, n_nodes, n_terms, n_coefs, n_words};
    fp2 nv[ir::MAX_NODES];
    fp2 r = ir::eval(s, words, reinterpret_cast<const fp2*>(coefs), reinterpret_cast<const fp2*>(values), nv);
    out[0] = r.c0;
    out[1] = r.c1;
}

// The evaluation plan the kernels run, thread form: built from the same word stream, then walked by one worker at one
// point.  Returns the plan builder's code (0 = built).
extern "C" int emul_ir_plan_eval(const u32* words, u32 n_words, u32 n_tables, u32 n_nodes, u32 n_terms, const u64* coefs, u32 n_coefs,
                                 const u64* values, u32 degree, u64* out, u32* plan_info /* sum levels, nodes, units, words, affine nodes */) {
    ir::Shape s{n_tables, n_nodes, n_terms, n_coefs, n_words};
    std::vector<u32> pw;
    if (int why = ir::build_plan(s, words, degree, pw)) return why;
    plan_info[0] = pw[0]; plan_info[1] = pw[1]; plan_info[2] = pw[2]; plan_info[3] = pw[8]; plan_info[4] = pw[9];
    std::vector<fp2> nv(pw[1], f2(0xA5A5A5A5A5A5A5A5ull, 0x5A5A5A5A5A5A5A5Aull));  // poisoned: a read before the write shows
    fp2 r = ir::plan_eval(pw.data(), reinterpret_cast<const fp2*>(coefs), reinterpret_cast<const fp2*>(values), nv.data());
    out[0] = r.c0;
    out[1] = r.c1;
    return 0;
}

// The pair form of a round: the polynomial at the points 0..=degree of one pair (lo = T(i), hi = T(i+half)) by `lanes`
// cooperating workers, the lanes of every phase run one after another.  With skip_one the point 1 is not evaluated
// (its output stays zero).
extern "C" int emul_ir_pair(const u32* words, u32 n_words, u32 n_tables, u32 n_nodes, u32 n_terms, const u64* coefs, u32 n_coefs,
                            const u64* lo, const u64* hi, u32 degree, u32 lanes, int skip_one, u64* out /* (degree + 1) x 2 */) {
    ir::Shape s{n_tables, n_nodes, n_terms, n_coefs, n_words};
    std::vector<u32> pw;
    if (int why = ir::build_plan(s, words, degree, pw)) return why;
    const u32 np = pw[16] + 1;  // the points the kernels evaluate: 0 .. min(declared, attained degree)
    const fp2 poison = f2(0xA5A5A5A5A5A5A5A5ull, 0x5A5A5A5A5A5A5A5Aull);
    const u32 ids = n_tables + pw[1];
    std::vector<fp2> area(ir::pair_area(n_tables, pw[1], np), poison);
    ir::Pair a;
    a.pw = pw.data(); a.cf = reinterpret_cast<const fp2*>(coefs);
    a.V = area.data(); a.DV = a.V + (size_t)ids * np; a.UB = a.DV + ids;
    a.n_tables = n_tables; a.np = np; a.npe = skip_one ? np - 1 : np;
    for (u32 t = 0; t < n_tables; t++) {
        a.V[t * np] = f2(lo[2 * t], lo[2 * t + 1]);
        a.DV[t] = f2_sub(f2(hi[2 * t], hi[2 * t + 1]), a.V[t * np]);
    }
    for (u32 g = 0; g < pw[11]; g++) {
        for (u32 l = 0; l < lanes; l++) ir::pair_affine_units(a, g, l, lanes);
        for (u32 l = 0; l < lanes; l++) ir::pair_affine_nodes(a, g, l, lanes);
    }
    for (u32 l = 0; l < lanes; l++) ir::pair_step(a, l, lanes);
    for (u32 lv = 0; lv < pw[0]; lv++) {
        for (u32 l = 0; l < lanes; l++) ir::pair_level_units(a, lv, l, lanes);
        for (u32 l = 0; l < lanes; l++) ir::pair_level_nodes(a, lv, l, lanes);
    }
    const u32 fin = (n_tables + pw[1] - 1) * np;
    for (u32 d = 0; d < 2 * (degree + 1); d++) out[d] = 0;
    for (u32 pi = 0; pi < a.npe; pi++) {
        const fp2 v = a.V[fin + a.point(pi)];
        out[2 * a.point(pi)] = v.c0;
        out[2 * a.point(pi) + 1] = v.c1;
    }
    return 0;
}

// The thread pair form: one worker, one pair, every point, compact values (live tables and nodes only).
extern "C" int emul_ir_tpair(const u32* words, u32 n_words, u32 n_tables, u32 n_nodes, u32 n_terms, const u64* coefs, u32 n_coefs,
                             const u64* lo, const u64* hi, u32 degree, int all_points /* 0 point by point, 1 all at once, 2 all but 1 */,
                             u64* out /* (degree + 1) x 2 */) {
    ir::Shape s{n_tables, n_nodes, n_terms, n_coefs, n_words};
    std::vector<u32> pw;
    if (int why = ir::build_plan(s, words, degree, pw)) return why;
    const fp2* cf = reinterpret_cast<const fp2*>(coefs);
    const fp2 poison = f2(0xA5A5A5A5A5A5A5A5ull, 0x5A5A5A5A5A5A5A5Aull);
    const u32 nl = pw[14];
    std::vector<fp2> V(nl + pw[1], poison), D(nl + pw[1], poison);
    const u32* live = pw.data() + pw[13];
    for (u32 j = 0; j < nl; j++) {
        V[j] = f2(lo[2 * live[j]], lo[2 * live[j] + 1]);
        D[j] = f2_sub(f2(hi[2 * live[j]], hi[2 * live[j] + 1]), V[j]);
    }
    ir::tpair_affine(pw.data(), cf, V.data(), D.data(), [&](u32 t, fp2& l, fp2& df) {
        l = f2(lo[2 * t], lo[2 * t + 1]);
        df = f2_sub(f2(hi[2 * t], hi[2 * t + 1]), l);
    });
    for (u32 d = 0; d < 2 * (degree + 1); d++) out[d] = 0;
    if (all_points) {  // unit by unit, every point at once
        if (!ir::tpair_all_fits(pw.data())) return -1;
        std::vector<fp2> W((size_t)ir::TPAIR_SUM_NODES * ir::TPAIR_POINTS, poison);
        fp2 res[ir::TPAIR_POINTS];
        ir::tpair_sums_all(pw.data(), cf, V.data(), D.data(), W.data(), all_points == 2, res);
        for (u32 d = 0; d <= pw[16]; d++) { out[2 * d] = res[d].c0; out[2 * d + 1] = res[d].c1; }
        return 0;
    }
    for (u32 d = 0; d <= pw[16]; d++) {
        if (d) ir::tpair_step(pw.data(), V.data(), D.data());
        const fp2 v = ir::tpair_sums(pw.data(), cf, V.data());
        out[2 * d] = v.c0;
        out[2 * d + 1] = v.c1;
    }
    return 0;
}
