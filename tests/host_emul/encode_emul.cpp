// Host-side execution of the row encoder's phase functions (csrc/encode_core.cuh), one
// emulated thread at a time.  Test infrastructure: it checks the kernels' index arithmetic
// (windows, swizzle, twiddle indexing, pad placement) on a machine without a GPU.  A phase is
// run for every thread before the next phase starts, which is what the barriers guarantee.
#include <cstdlib>
#include <cstring>
#include <vector>
#include "../../intelligenceregulation_b200/csrc/encode_core.cuh"

using namespace enc;

static std::vector<u64> make_tw(u32 lognn) {
    u64 r32 = gl_pow(7, (GL_P - 1) >> 32), w = gl_pow(r32, 1ULL << (32 - lognn));
    std::vector<u64> tw((size_t)1 << lognn);
    u64 c = 1;
    for (auto& x : tw) { x = c; c = gl_mul(c, w); }
    return tw;
}

struct NoSync { void operator()() const {} };

template <int LOGN>
static void run_fast(RowArgs a, u32 nt) {
    using F = Fast<LOGN>;
    std::vector<u64> S(F::N + 16), TW(F::TW_WORDS + 16);
    for (u32 t = 0; t < nt; t++) F::load_twiddles(a, TW.data(), t, nt);
    // one emulated thread owning every group keeps the pass order of the device code
    for (u32 row = 0; row < a.rows; row++) {
        F::row_coeffs(a, row, S.data(), TW.data(), a.scratch, 0, 1, NoSync());
        for (u32 s = 0; s < (1u << a.logr); s++) F::row_residue(a, row, s, S.data(), TW.data(), a.scratch, 0, 1, NoSync());
    }
}

extern "C" int emul_encode(int fast, const u64* data, u32 rows, u32 logn, u32 logr, const u64* pads, u32 q,
                           const u64* pows, int zk, u32 nt, u64* out) {
    u32 n = 1u << logn;
    std::vector<u64> tw = make_tw(logn + logr);
    // rows above 2^14 words run as 2 or 4 transforms of 2^14, exactly as the library's commit sets them up
    const u32 logb = logn > 14 ? 14 : logn, loga = logn - logb, nb = 1u << logb;
    RowArgs a;
    a.data = data; a.pads = pads; a.pows = pows; a.tw_nn = tw.data(); a.enc = out;
    a.rows = rows; a.q = zk ? q : 0; a.logr = logr + loga; a.loga = loga; a.zk = zk;
    a.T = zk ? (n + q + nb - 1) / nb : n / nb;
    a.ninv = gl_inv(n); a.coef_out = nullptr; a.split = 0;
    std::vector<u64> X((size_t)a.T * nb, 0xA5A5A5A5A5A5A5A5ULL);  // poisoned: unwritten words must never be read
    a.scratch = X.data();
    if (fast) {
        switch (logb) {
            case 8: run_fast<8>(a, nt); break;
            case 9: run_fast<9>(a, nt); break;
            case 10: run_fast<10>(a, nt); break;
            case 11: run_fast<11>(a, nt); break;
            case 12: run_fast<12>(a, nt); break;
            case 13: run_fast<13>(a, nt); break;
            case 14: run_fast<14>(a, nt); break;
            default: return -1;
        }
        return 0;
    }
    std::vector<u64> S(n);
    for (u32 row = 0; row < rows; row++) {
        for (u32 t = 0; t < nt; t++) Generic::load(a, row, logn, S.data(), t, nt);
        for (u32 ln = logn; ln >= 1; ln--)
            for (u32 t = 0; t < nt; t++) Generic::dif_stage(a, logn, ln, S.data(), t, nt);
        for (u32 t = 0; t < nt; t++) Generic::coeffs(a, row, logn, S.data(), a.scratch, t, nt);
        for (u32 s = 0; s < (1u << logr); s++) {
            for (u32 t = 0; t < nt; t++) Generic::twist(a, logn, s, a.scratch, S.data(), t, nt);
            for (u32 ln = 1; ln <= logn; ln++)
                for (u32 t = 0; t < nt; t++) Generic::dit_stage(a, logn, ln, S.data(), t, nt);
            for (u32 t = 0; t < nt; t++) Generic::store(a, row, logn, s, S.data(), t, nt);
        }
    }
    return 0;
}
