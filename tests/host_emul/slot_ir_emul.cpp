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
