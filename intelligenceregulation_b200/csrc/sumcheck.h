// Shared declarations of the sumcheck kernels and their C-ABI wrapper.
#pragma once
#include <cuda_runtime.h>
#include "gl_field.cuh"
#include "slot_ir.cuh"

namespace hlk {

enum { POLY_PROD = 0, POLY_ZC = 1, POLY_LOGUP_Q = 2, POLY_LOGUP_T = 3, POLY_IR = 4 };
constexpr int SC_MAX_POINTS = 8;  // degree <= 7

// Device-resident state of one evaluator: the transcript (state, counter, key), the running
// unmasked claim, the last challenge, and the CFS mask's running terms.
struct ScState {
    uint32_t state[8];
    uint32_t key[8];
    u64 counter;
    int keyed;
    int pad_;
    fp2 claim;
    fp2 r;
    fp2 mask_c;
    fp2 acc_prev;   // sum_{i<j} u_i(r_i)
    fp2 ap;         // a' prod_{i<j} r_i (the mask's linear term, sumcheck.rs:260-295)
};

struct ScStep {
    const u64* partials;        // nblocks x (degree+1) Fp2
    u32 nblocks;
    int degree, round;
    int use_claim;              // s(1) := claim - s(0)
    int recover;                // keep the running claim (rounds.rs recover_one)
    int fs;                     // 0: only reduce and write the sums (host-driven round())
    const u64* mask;            // CFS coefficients [a0, a', a_{j,e}] or NULL
    // per round j and point x = 0..degree: 2^(N-1-j) (a0 + sum_{i>j} u_i(1)/2 + u_j(x)), the part of the mask's round
    // polynomial g_j(x) that no challenge enters (made by the host once per batch)
    const u64* mask_tab;
    const u64* mask_row = nullptr;  // when set: this round's `degree` coefficients a_{j,e} and (tab_row) its degree+1 table entries, already picked out
    const u64* tab_row = nullptr;
    int mask_vars;
    const u64* inv_den;         // degree+1 inverse Lagrange denominators
    int eval_degree;            // the sums arrive at the points 0..eval_degree; the points above are extrapolated
    const u64* extrap;          // (degree - eval_degree) rows of eval_degree + 1 base-field weights, or NULL
    ScState* state;
    u64* out;                   // per round: (degree+1) sums, (degree+1) masked, r  (Fp2 each)
};

// a slot polynomial given as data (slot_ir.cuh), resident on the device
struct IrDev {
    const u32* plan;   // the evaluation plan (slot_ir.cuh)
    const u64* coefs;  // n_coefs Fp2
    u32 plan_words, n_coefs, n_tables, n_nodes /* with the final one */, n_units;
    u32 eval_degree;   // min(declared, attained): the points the kernels evaluate are 0 .. eval_degree
    int all_points;    // the plan fits the thread pair form that evaluates a unit at every point at once
};

void sc_set_dependent_launch(bool on);
u32 sc_round_blocks(u32 half, int sm_count);
// the data-driven evaluator: one CTA row per evaluation point, `sc_ir_blocks` CTAs per row
u32 sc_ir_blocks(const IrDev& p, u32 half, int degree, int sm_count);
u32 sc_ir_max_blocks(u32 half, int sm_count);
u32 sc_ir_tail_len(const IrDev& p, int degree);
bool sc_ir_fits(const IrDev& p, int degree);  // the pair form's areas fit one CTA's shared memory
cudaError_t sc_round_ir(const IrDev& p, int k, const u64* tables, size_t stride, u32 half, int degree, int eval_one, u64* partials,
                        u32 nblocks, cudaStream_t s);
cudaError_t sc_tail_ir(const IrDev& p, int k, u64* tables, size_t stride, u32 len, int degree, const ScStep& a, int nrounds,
                       int first_has_claim, cudaStream_t s);
bool sc_supported(int poly, int k, int degree);
cudaError_t sc_round(int poly, int k, const u64* tables, size_t stride, u32 half, const u64* coefs, int eval_one, u64* partials,
                     u32 nblocks, cudaStream_t s);
cudaError_t sc_step(const ScStep& a, cudaStream_t s);
// closed-form families: fold with the challenge in `st` and sum the next round (length n after the fold) in one pass
cudaError_t sc_fold_round(int poly, int k, u64* tables, size_t stride, u32 n, const u64* coefs, const ScState* st, int eval_one, u64* partials,
                          u32 nblocks, cudaStream_t s);
constexpr u32 SC_TAIL_LEN = 2048;  // table length from which the remaining rounds run in one CTA (measured on the 3-table degree-3 family: 1024 -> 0.467 ms, 2048 -> 0.450, 4096 -> 0.480, 8192 -> 0.517 for 21 rounds; above it the arithmetic of one SM costs more than the launches it saves)
cudaError_t sc_tail(int poly, int k, u64* tables, size_t stride, u32 len, const u64* coefs, const ScStep& a, int nrounds,
                    int first_has_claim, u64* scratch, cudaStream_t s);
// bit t of *d_mask is set when table t holds a non-zero second word anywhere in its first `len` entries (*d_mask zeroed by the caller)
cudaError_t sc_nonbase_mask(const u64* tables, size_t stride, size_t len, u32 k, u64* d_mask, int sm_count, cudaStream_t s);
cudaError_t sc_fold(u64* tables, size_t stride, u32 half, u32 k, const ScState* st, cudaStream_t s);

}  // namespace hlk
