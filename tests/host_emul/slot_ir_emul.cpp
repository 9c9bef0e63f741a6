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

// The evaluation plan the kernels run: built from the same word stream, then evaluated either by one worker
// (`lanes` == 0, the thread form) or level by level with `lanes` workers run one after another (the warp form).
// Returns the plan builder's code (0 = built).
extern "C" int emul_ir_plan_eval(const u32* words, u32 n_words, u32 n_tables, u32 n_nodes, u32 n_terms, const u64* coefs, u32 n_coefs,
                                 const u64* values, u32 lanes, u64* out, u32* plan_info /* levels, nodes, units, words */) {
    ir::Shape s{n_tables, n_nodes, n_terms, n_coefs, n_words};
    std::vector<u32> pw;
    if (int why = ir::build_plan(s, words, pw)) return why;
    plan_info[0] = pw[0]; plan_info[1] = pw[1]; plan_info[2] = pw[2]; plan_info[3] = pw[8];
    const fp2* cf = reinterpret_cast<const fp2*>(coefs);
    const fp2* tv = reinterpret_cast<const fp2*>(values);
    std::vector<fp2> nv(pw[1]), ub(ir::PLAN_LEVEL_UNITS);
    for (auto& x : nv) x = f2(0xA5A5A5A5A5A5A5A5ull, 0x5A5A5A5A5A5A5A5Aull);  // poisoned: a read before the write shows
    for (auto& x : ub) x = f2(0xA5A5A5A5A5A5A5A5ull, 0x5A5A5A5A5A5A5A5Aull);
    fp2 r;
    if (lanes == 0) {
        r = ir::plan_eval(pw.data(), cf, tv, nv.data());
    } else {
        for (u32 l = 0; l < pw[0]; l++) {
            for (u32 lane = 0; lane < lanes; lane++) ir::plan_level_units(pw.data(), l, cf, tv, nv.data(), ub.data(), lane, lanes);
            for (u32 lane = 0; lane < lanes; lane++) ir::plan_level_nodes(pw.data(), l, ub.data(), nv.data(), lane, lanes);
        }
        r = nv[pw[1] - 1];
    }
    out[0] = r.c0;
    out[1] = r.c1;
    return 0;
}
