// C ABI: the sumcheck evaluator (`impl SumcheckRounds`, sumcheck/rounds.rs:22-28) and its
// device-side batch of rounds with the Fiat-Shamir step (the reference's Metal form:
// metal.rs:3509-3669 MetalRounds, :4141-4192 TailedRounds::masked_prove).
#include <cstring>

#include "api_internal.h"
#include "../../include/hl_b200_bench.h"
#include "slot_gen.cuh"
#include "sumcheck.h"

using namespace hlapi;

struct hl_tables;
u64* hl_tables_adopt(hl_tables* t);        // tables.cu: hands the device tables over (the set is empty afterwards)
const u64* hl_tables_peek(hl_tables* t);   // the device tables, still owned by the set
int hl_tables_flush_locked(hl_tables* t);  // waits for the builders; refuses a base-declared table with an extension word
void hl_tables_shape(hl_tables* t, hl_ctx** c, size_t* k, uint32_t* n_vars);

struct hl_rounds {
    hl_ctx* ctx = nullptr;
    int poly = 0;
    u32 k = 0, n_vars = 0, degree = 0, next = 0;
    size_t stride = 0, len = 0, ncoefs = 0;
    u32 max_blocks = 0;
    u64* d_tables = nullptr;
    u64* d_coefs = nullptr;
    u64* d_partials = nullptr;
    u64* d_out = nullptr;      // n_vars rows of (2 (degree+1) + 1) Fp2
    u64* d_inv_den = nullptr;
    u64* d_extrap = nullptr;   // weights of the points above the evaluated degree (data-form polynomials only)
    u32 eval_degree = 0;
    hlk::ScState* d_state = nullptr;
    hlk::IrDev ir{};           // poly == POLY_IR: the polynomial as data
    const sg::Entry* gen = nullptr;  // the generated kernel of this program's graph, when there is one
    u64* d_cfo = nullptr;      // its coefficients by occurrence
    u64* d_nonbase = nullptr;  // one word: bit t set when table t is extension-valued before the first fold
    u64 nonbase = ~0ull;
    u32 tail_len = hlk::SC_TAIL_LEN;
    size_t out_row() const { return (2 * ((size_t)degree + 1) + 1) * 2; }
};

namespace {

void free_rounds(hl_rounds* r) {
    hl_ctx* c = r->ctx;
    if (r->d_tables) dev_free(c, r->d_tables, r->k * r->stride * 16);
    dev_free(c, r->d_coefs, (r->ncoefs ? r->ncoefs : 1) * 16);
    dev_free(c, r->d_partials, (size_t)r->max_blocks * (r->degree + 1) * 16);
    dev_free(c, r->d_out, (r->n_vars ? r->n_vars : 1) * r->out_row() * 8);
    dev_free(c, r->d_inv_den, ((size_t)r->degree + 1) * 8);
    if (r->d_extrap) dev_free(c, r->d_extrap, (size_t)hlk::SC_MAX_POINTS * hlk::SC_MAX_POINTS * 8);
    dev_free(c, r->d_state, sizeof(hlk::ScState));
    if (r->d_cfo) dev_free(c, r->d_cfo, (size_t)(r->gen ? r->gen->n_cfo : 1) * 16);
    if (r->d_nonbase) dev_free(c, r->d_nonbase, 8);
    if (r->ir.plan) dev_free(c, (void*)r->ir.plan, (size_t)r->ir.plan_words * 4);
    if (r->ir.coefs) dev_free(c, (void*)r->ir.coefs, (size_t)(r->ir.n_coefs ? r->ir.n_coefs : 1) * 16);
    delete r;
}

// the reduce + Fiat-Shamir step of round r->next over `nb` partial rows
int launch_step(hl_rounds* r, u32 nb, int fs, int use_claim, int recover, const u64* d_mask, const u64* d_mtab, int mask_vars) {
    hl_ctx* c = r->ctx;
    hlk::ScStep a;
    a.partials = r->d_partials; a.nblocks = nb; a.degree = (int)r->degree; a.round = (int)r->next;
    a.use_claim = use_claim; a.recover = recover; a.fs = fs; a.mask = d_mask; a.mask_tab = d_mtab; a.mask_vars = mask_vars;
    a.inv_den = r->d_inv_den; a.state = r->d_state; a.out = r->d_out;
    a.eval_degree = (int)r->eval_degree; a.extrap = r->d_extrap;
    cudaError_t e = hlk::sc_step(a, c->stream);
    c->stats.kernel_launches++;
    if (e != cudaSuccess) return fail(c, HL_B200_ERR_DEVICE, "round step launch", e);
    return HL_B200_OK;
}

// launches round j's kernels; the caller holds the context lock
int launch_round(hl_rounds* r, int eval_one, int fs, int use_claim, int recover, const u64* d_mask, const u64* d_mtab, int mask_vars) {
    hl_ctx* c = r->ctx;
    const u32 half = (u32)(r->len / 2);
    const bool is_ir = r->poly == hlk::POLY_IR;
    u32 nb = is_ir ? hlk::sc_ir_blocks(r->ir, half, (int)r->degree, c->sm_count) : hlk::sc_round_blocks(half, c->sm_count);
    if (nb > r->max_blocks) return fail(c, HL_B200_ERR_DEVICE, "round launch: more partial rows than the buffer holds");  // the two grid rules agree by construction
    cudaError_t e;
    if (is_ir && r->gen && c->slot_kernels) {
        // the generated kernel of this graph: the first-round typing while the tables it reads as base words are base-valued
        const u32 skip = (!eval_one && r->eval_degree >= 1) ? 1u : 0u, npe = r->eval_degree + 1 - skip;
        const bool r0 = r->next == 0 && (r->gen->base_mask & r->nonbase) == 0;
        const bool per_point = (u64)half < (u64)c->sm_count * sg::GT * 2;
        u32 bx = (half + sg::GT - 1) / sg::GT, cap = (u32)c->sm_count * 4;
        if (bx > cap) bx = cap;
        if (bx > r->max_blocks) bx = r->max_blocks;
        if (bx < 1) bx = 1;
        nb = bx;
        c->stats.generated_rounds++;
        e = r->gen->launch(r0, per_point, bx, r->d_tables, r->stride, half, r->d_cfo, (int)r->degree, npe, skip, r->d_partials, c->stream);
    } else {
        e = is_ir ? hlk::sc_round_ir(r->ir, (int)r->k, r->d_tables, r->stride, half, (int)r->degree, eval_one, r->d_partials, nb, c->stream)
                  : hlk::sc_round(r->poly, (int)r->k, r->d_tables, r->stride, half, r->d_coefs, eval_one, r->d_partials, nb, c->stream);
    }
    c->stats.kernel_launches++;
    if (e != cudaSuccess) return fail(c, HL_B200_ERR_DEVICE, "round launch", e);
    return launch_step(r, nb, fs, use_claim, recover, d_mask, d_mtab, mask_vars);
}

int launch_fold(hl_rounds* r) {
    hl_ctx* c = r->ctx;
    cudaError_t e = hlk::sc_fold(r->d_tables, r->stride, (u32)(r->len / 2), r->k, r->d_state, c->stream);
    c->stats.kernel_launches++;
    if (e != cudaSuccess) return fail(c, HL_B200_ERR_DEVICE, "fold launch", e);
    r->len /= 2;
    r->next++;
    return HL_B200_OK;
}

}  // namespace

extern "C" {

}  // extern "C"

namespace {

// the evaluator of either kind; `words` is the data form of the polynomial when poly == POLY_IR
constexpr size_t FUSED_FOLD_MAX_PAIRS = (size_t)1 << 15;

struct GenAsk {  // a slot program's generated kernel, looked up by the caller
    const sg::Entry* entry = nullptr;
    std::vector<fp2> cfo;
};

int rounds_build(hl_ctx* c, int poly, size_t k, uint32_t n_vars, uint32_t degree, const uint64_t* tables, const uint64_t* coefs,
                 size_t ncoefs, const std::vector<u32>* plan, hl_rounds** out, hl_tables* built = nullptr, const GenAsk* gen = nullptr) {
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    if (built) {
        if (int rc = hl_tables_flush_locked(built)) return rc;
    }
    hl_rounds* r = new hl_rounds();
    r->ctx = c; r->poly = poly; r->k = (u32)k; r->n_vars = n_vars; r->degree = degree; r->ncoefs = ncoefs;
    r->stride = r->len = (size_t)1 << n_vars;
    r->max_blocks = hlk::sc_round_blocks((u32)(r->len / 2), c->sm_count);
    r->eval_degree = degree;
    if (poly == hlk::POLY_IR) {
        const std::vector<u32>& pw = *plan;
        r->eval_degree = r->ir.eval_degree = pw[16];
        r->ir.all_points = ir::tpair_all_fits(pw.data()) ? 1 : 0;
        r->ir.plan_words = (u32)pw.size(); r->ir.n_coefs = (u32)ncoefs; r->ir.n_tables = (u32)k;
        r->ir.n_nodes = pw[1]; r->ir.n_units = pw[2];
        if (!hlk::sc_ir_fits(r->ir, (int)degree)) {
            delete r;
            return fail(c, HL_B200_ERR_UNSUPPORTED, "slot program: tables x nodes x points beyond one CTA's shared memory");
        }
        r->max_blocks = hlk::sc_ir_max_blocks((u32)(r->len / 2), c->sm_count);
        r->tail_len = hlk::sc_ir_tail_len(r->ir, (int)degree);
    }
    u64 inv_den[hlk::SC_MAX_POINTS];
    for (u32 i = 0; i <= degree; i++) {
        u64 den = 1;
        for (u32 j = 0; j <= degree; j++)
            if (j != i) den = gl_mul(den, gl_from_i64((long long)i - (long long)j));
        inv_den[i] = gl_inv(den);
    }
    int rc = built ? HL_B200_OK : dev_alloc(c, (void**)&r->d_tables, k * r->stride * 16);
    if (!rc) rc = dev_alloc(c, (void**)&r->d_coefs, (ncoefs ? ncoefs : 1) * 16);
    if (!rc) rc = dev_alloc(c, (void**)&r->d_partials, (size_t)r->max_blocks * (degree + 1) * 16);
    if (!rc) rc = dev_alloc(c, (void**)&r->d_out, (n_vars ? n_vars : 1) * r->out_row() * 8);
    if (!rc) rc = dev_alloc(c, (void**)&r->d_inv_den, ((size_t)degree + 1) * 8);
    if (!rc) rc = dev_alloc(c, (void**)&r->d_state, sizeof(hlk::ScState));
    if (!rc && !built) rc = h2d(c, r->d_tables, tables, k * r->stride * 16);
    if (!rc && ncoefs) rc = h2d(c, r->d_coefs, coefs, ncoefs * 16);
    if (!rc) rc = h2d(c, r->d_inv_den, inv_den, ((size_t)degree + 1) * 8);
    if (!rc && r->eval_degree < degree) {
        // s(p) = sum_i s(i) prod_{j != i} (p - j) / (i - j) over i, j <= eval_degree, for p above it
        u64 wts[hlk::SC_MAX_POINTS * hlk::SC_MAX_POINTS] = {0};
        const u32 de = r->eval_degree;
        for (u32 pnt = de + 1; pnt <= degree; pnt++)
            for (u32 i = 0; i <= de; i++) {
                u64 num = 1, den = 1;
                for (u32 j = 0; j <= de; j++)
                    if (j != i) {
                        num = gl_mul(num, gl_from_i64((long long)pnt - (long long)j));
                        den = gl_mul(den, gl_from_i64((long long)i - (long long)j));
                    }
                wts[(pnt - de - 1) * (de + 1) + i] = gl_mul(num, gl_inv(den));
            }
        rc = dev_alloc(c, (void**)&r->d_extrap, sizeof wts);
        if (!rc) rc = h2d(c, r->d_extrap, wts, sizeof wts);
    }
    if (!rc && poly == hlk::POLY_IR) {
        rc = dev_alloc(c, (void**)&r->ir.plan, (size_t)r->ir.plan_words * 4);
        if (!rc) rc = dev_alloc(c, (void**)&r->ir.coefs, (size_t)(ncoefs ? ncoefs : 1) * 16);
        if (!rc) rc = h2d(c, (void*)r->ir.plan, plan->data(), (size_t)r->ir.plan_words * 4);
        if (!rc && ncoefs) rc = h2d(c, (void*)r->ir.coefs, coefs, ncoefs * 16);
    }
    if (!rc) {
        cudaError_t e = cudaMemsetAsync(r->d_state, 0, sizeof(hlk::ScState), c->stream);
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "state clear", e);
    }
    if (!rc && c->slot_kernels && gen && gen->entry && gen->entry->n_tables == k && gen->entry->n_cfo == gen->cfo.size()) {
        // the generated kernels are switched on and the graph has one: its coefficients by occurrence, and which tables are base-valued
        // right now (a scan of every table: not paid while the switch is off)
        r->gen = gen->entry;
        rc = dev_alloc(c, (void**)&r->d_cfo, (size_t)(gen->cfo.size() ? gen->cfo.size() : 1) * 16);
        if (!rc) rc = dev_alloc(c, (void**)&r->d_nonbase, 8);
        if (!rc && gen->cfo.size()) rc = h2d(c, r->d_cfo, gen->cfo.data(), gen->cfo.size() * 16);
        if (!rc && cudaMemsetAsync(r->d_nonbase, 0, 8, c->stream) != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "mask clear");
        if (!rc) {
            const u64* tabs = built ? hl_tables_peek(built) : r->d_tables;
            cudaError_t e = hlk::sc_nonbase_mask(tabs, r->stride, r->len, (u32)k, r->d_nonbase, c->sm_count, c->stream);
            c->stats.kernel_launches++;
            if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "table typing launch", e);
        }
        if (!rc) rc = d2h(c, &r->nonbase, r->d_nonbase, 8);
    }
    if (!rc) rc = sync(c, "rounds_new");
    if (rc) { cudaStreamSynchronize(c->stream); free_rounds(r); return rc; }
    if (built) r->d_tables = hl_tables_adopt(built);  // only now: a failed build leaves the set with its owner
    *out = r;
    return HL_B200_OK;
}

}  // namespace

extern "C" {

int hl_b200_rounds_new(hl_ctx* c, int poly, size_t k, uint32_t n_vars, uint32_t degree, const uint64_t* tables,
                       const uint64_t* coefs, size_t ncoefs, hl_rounds** out) {
    if (!c || !tables || !out) return fail(c, HL_B200_ERR_ARG, "rounds_new: null argument");
    if (n_vars > 30) return fail(c, HL_B200_ERR_UNSUPPORTED, "rounds_new: more than 30 variables");
    if (poly == hlk::POLY_IR) return fail(c, HL_B200_ERR_ARG, "rounds_new: a data-form polynomial goes through rounds_new_ir");
    if (!hlk::sc_supported(poly, (int)k, (int)degree)) return fail(c, HL_B200_ERR_UNSUPPORTED, "rounds_new: polynomial family / table count / degree");
    if ((poly == hlk::POLY_LOGUP_Q || poly == hlk::POLY_LOGUP_T) && (!coefs || ncoefs < 1)) return fail(c, HL_B200_ERR_ARG, "rounds_new: alpha missing");
    return rounds_build(c, poly, k, n_vars, degree, tables, coefs, ncoefs, nullptr, out);
}

int hl_b200_rounds_new_ir(hl_ctx* c, size_t k, uint32_t n_vars, uint32_t degree, const uint64_t* tables, const uint32_t* words,
                          size_t n_words, uint32_t n_nodes, uint32_t n_terms, const uint64_t* coefs, size_t ncoefs, hl_rounds** out) {
    if (!c || !tables || !words || !out || (ncoefs && !coefs)) return fail(c, HL_B200_ERR_ARG, "rounds_new_ir: null argument");
    if (n_vars > 30) return fail(c, HL_B200_ERR_UNSUPPORTED, "rounds_new_ir: more than 30 variables");
    if (!hlk::sc_supported(hlk::POLY_IR, (int)k, (int)degree) || n_words > ir::MAX_WORDS || n_nodes > ir::MAX_NODES || ncoefs > ir::MAX_COEFS)
        return fail(c, HL_B200_ERR_UNSUPPORTED, "rounds_new_ir: table count, degree or program size beyond the evaluator's limits");
    ir::Shape sh{(u32)k, n_nodes, n_terms, (u32)ncoefs, (u32)n_words};
    if (int why = ir::validate(sh, words)) {
        char buf[96];
        snprintf(buf, sizeof buf, "rounds_new_ir: malformed program (check %d)", why);
        return fail(c, HL_B200_ERR_ARG, buf);
    }
    std::vector<u32> plan;
    if (int why = ir::build_plan(sh, words, degree, plan)) {
        char buf[96];
        snprintf(buf, sizeof buf, "rounds_new_ir: the program does not fit the evaluator's plan (reason %d)", why);
        return fail(c, HL_B200_ERR_UNSUPPORTED, buf);
    }
    GenAsk gen;
    gen.entry = sg::find(ir::signature(sh, words, reinterpret_cast<const fp2*>(coefs), &gen.cfo));
    return rounds_build(c, hlk::POLY_IR, k, n_vars, degree, tables, coefs, ncoefs, &plan, out, nullptr, &gen);
}

int hl_b200_rounds_from_tables(hl_ctx* c, int poly, uint32_t degree, hl_tables* t, const uint64_t* coefs, size_t ncoefs, hl_rounds** out) {
    if (!c || !t || !out) return fail(c, HL_B200_ERR_ARG, "rounds_from_tables: null argument");
    hl_ctx* tc = nullptr;
    size_t k = 0;
    uint32_t n_vars = 0;
    hl_tables_shape(t, &tc, &k, &n_vars);
    if (tc != c || k == 0) return fail(c, HL_B200_ERR_ARG, "rounds_from_tables: the table set is empty or belongs to another context");
    if (poly == hlk::POLY_IR) return fail(c, HL_B200_ERR_ARG, "rounds_from_tables: a data-form polynomial goes through rounds_from_tables_ir");
    if (!hlk::sc_supported(poly, (int)k, (int)degree)) return fail(c, HL_B200_ERR_UNSUPPORTED, "rounds_from_tables: polynomial family / table count / degree");
    if ((poly == hlk::POLY_LOGUP_Q || poly == hlk::POLY_LOGUP_T) && (!coefs || ncoefs < 1)) return fail(c, HL_B200_ERR_ARG, "rounds_from_tables: alpha missing");
    return rounds_build(c, poly, k, n_vars, degree, nullptr, coefs, ncoefs, nullptr, out, t);
}

int hl_b200_rounds_from_tables_ir(hl_ctx* c, uint32_t degree, hl_tables* t, const uint32_t* words, size_t n_words, uint32_t n_nodes,
                                  uint32_t n_terms, const uint64_t* coefs, size_t ncoefs, hl_rounds** out) {
    if (!c || !t || !words || !out || (ncoefs && !coefs)) return fail(c, HL_B200_ERR_ARG, "rounds_from_tables_ir: null argument");
    hl_ctx* tc = nullptr;
    size_t k = 0;
    uint32_t n_vars = 0;
    hl_tables_shape(t, &tc, &k, &n_vars);
    if (tc != c || k == 0) return fail(c, HL_B200_ERR_ARG, "rounds_from_tables_ir: the table set is empty or belongs to another context");
    if (!hlk::sc_supported(hlk::POLY_IR, (int)k, (int)degree) || n_words > ir::MAX_WORDS || n_nodes > ir::MAX_NODES || ncoefs > ir::MAX_COEFS)
        return fail(c, HL_B200_ERR_UNSUPPORTED, "rounds_from_tables_ir: table count, degree or program size beyond the evaluator's limits");
    ir::Shape sh{(u32)k, n_nodes, n_terms, (u32)ncoefs, (u32)n_words};
    if (ir::validate(sh, words)) return fail(c, HL_B200_ERR_ARG, "rounds_from_tables_ir: malformed program");
    std::vector<u32> plan;
    if (ir::build_plan(sh, words, degree, plan)) return fail(c, HL_B200_ERR_UNSUPPORTED, "rounds_from_tables_ir: the program does not fit the evaluator's plan");
    GenAsk gen;
    gen.entry = sg::find(ir::signature(sh, words, reinterpret_cast<const fp2*>(coefs), &gen.cfo));
    return rounds_build(c, hlk::POLY_IR, k, n_vars, degree, nullptr, coefs, ncoefs, &plan, out, t, &gen);
}

void hl_b200_rounds_free(hl_rounds* r) {
    if (!r) return;
    hl_ctx* c = r->ctx;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    free_rounds(r);
}

int hl_b200_rounds_round(hl_rounds* r, uint32_t j, int eval_one, uint64_t* sums) {
    if (!r || !sums) return HL_B200_ERR_ARG;
    hl_ctx* c = r->ctx;
    if (j != r->next || j >= r->n_vars) return fail(c, HL_B200_ERR_ARG, "rounds_round: round order (a round needs the preceding fold)");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    int rc;
    {
        Timed t(c, HL_T_ROUNDS);
        rc = launch_round(r, eval_one, 0, 0, 0, nullptr, nullptr, 0);
    }
    if (!rc) rc = d2h(c, sums, r->d_out + (size_t)j * r->out_row(), ((size_t)r->degree + 1) * 16);
    if (!rc) rc = sync(c, "rounds_round");
    return rc;
}

int hl_b200_rounds_fold(hl_rounds* r, const uint64_t rr[2]) {
    if (!r || !rr) return HL_B200_ERR_ARG;
    hl_ctx* c = r->ctx;
    if (r->next >= r->n_vars) return fail(c, HL_B200_ERR_ARG, "rounds_fold: every variable is already folded");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    int rc = h2d(c, (char*)r->d_state + offsetof(hlk::ScState, r), rr, 16);
    if (!rc) {
        Timed t(c, HL_T_ROUNDS);
        rc = launch_fold(r);
    }
    if (!rc) rc = sync(c, "rounds_fold");
    return rc;
}

int hl_b200_rounds_finals(hl_rounds* r, uint64_t* out) {
    if (!r || !out) return HL_B200_ERR_ARG;
    hl_ctx* c = r->ctx;
    if (r->next != r->n_vars) return fail(c, HL_B200_ERR_ARG, "rounds_finals: finals need all folds");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    int rc = HL_B200_OK;
    for (u32 t = 0; t < r->k && !rc; t++) rc = d2h(c, out + 2 * t, r->d_tables + 2 * (size_t)t * r->stride, 16);
    if (!rc) rc = sync(c, "rounds_finals");
    return rc;
}

int hl_b200_set_dependent_launch(int on) {
    hlk::sc_set_dependent_launch(on != 0);
    return HL_B200_OK;
}

int hl_b200_rounds_batched(hl_rounds* r, uint32_t nd, hl_fs_state* fs, const uint64_t* mask_coeffs, uint32_t mask_vars,
                           const uint64_t mask_c[2], uint64_t* out) {
    if (!r || !fs || !out) return HL_B200_ERR_ARG;
    hl_ctx* c = r->ctx;
    if (nd == 0) return HL_B200_OK;
    if (r->next + nd > r->n_vars) return fail(c, HL_B200_ERR_ARG, "rounds_batched: more rounds than variables left");
    if (mask_coeffs && (r->next != 0 || !mask_c || mask_vars < r->n_vars || mask_vars > 63))
        return fail(c, HL_B200_ERR_ARG, "rounds_batched: a masked batch starts at round 0 and its mask covers every variable");
    if (fs->recover_one && r->degree < 1) return fail(c, HL_B200_ERR_ARG, "rounds_batched: claim recovery requires degree >= 1");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    hlk::ScState st;
    memset(&st, 0, sizeof st);
    memcpy(st.state, fs->state, 32);
    memcpy(st.key, fs->key, 32);
    st.counter = fs->counter;
    st.keyed = fs->keyed;
    st.claim = f2(fs->claim[0], fs->claim[1]);
    u64 *d_mask = nullptr, *d_mtab = nullptr;
    const size_t mlen = mask_coeffs ? (size_t)mask_vars * r->degree + 2 : 0;
    const size_t tab_words = (size_t)mask_vars * (r->degree + 1) * 2;
    std::vector<u64> mtab;
    int rc = HL_B200_OK;
    if (mask_coeffs) {
        st.mask_c = f2(mask_c[0], mask_c[1]);
        const fp2* co = reinterpret_cast<const fp2*>(mask_coeffs);
        st.ap = co[1];  // a' times the empty product
        // per round j and point x: 2^(N-1-j) (a0 + sum_{i>j} u_i(1)/2 + u_j(x)) (sumcheck.rs:260-295): the part of g_j(x) no challenge enters
        const u64 half = gl_inv(2);
        mtab.assign(tab_words, 0);
        fp2 run = f2(0, 0);
        for (int i = (int)mask_vars - 1; i >= 0; i--) {
            const fp2* ai = co + 2 + (size_t)i * r->degree;
            const u64 scale = 1ull << (mask_vars - 1 - (u32)i);  // mask_vars <= 63: the power of two is its own canonical word
            for (u32 x = 0; x <= r->degree; x++) {
                fp2 u = f2(0, 0);
                u64 xp = 1;
                for (u32 e = 1; e <= r->degree; e++) { xp = gl_mul(xp, (u64)x); u = f2_add(u, f2_mul_base(ai[e - 1], xp)); }
                const fp2 v = f2_mul_base(f2_add(f2_add(co[0], run), u), scale);
                mtab[((size_t)i * (r->degree + 1) + x) * 2] = v.c0; mtab[((size_t)i * (r->degree + 1) + x) * 2 + 1] = v.c1;
            }
            fp2 u1 = f2(0, 0);
            for (u32 e = 0; e < r->degree; e++) u1 = f2_add(u1, ai[e]);
            run = f2_add(run, f2_mul_base(u1, half));
        }
        rc = dev_alloc(c, (void**)&d_mask, mlen * 16);
        if (!rc) rc = dev_alloc(c, (void**)&d_mtab, tab_words * 8);
        if (!rc) rc = h2d(c, d_mask, mask_coeffs, mlen * 16);
        if (!rc) rc = h2d(c, d_mtab, mtab.data(), tab_words * 8);
    }
    if (!rc) rc = h2d(c, r->d_state, &st, sizeof st);
    const u32 first = r->next;
    bool have_claim = fs->recover_one && fs->have_claim;
    {
        Timed t(c, HL_T_ROUNDS);
        u32 i = 0;
        if (r->poly == hlk::POLY_IR) {
            for (; i < nd && !rc && r->len > r->tail_len; i++) {
                rc = launch_round(r, have_claim ? 0 : 1, 1, have_claim ? 1 : 0, fs->recover_one ? 1 : 0, d_mask, d_mtab, (int)mask_vars);
                if (!rc) rc = launch_fold(r);
                have_claim = fs->recover_one != 0;
            }
        } else {
            // closed-form families: after the first long round the fold with the last challenge rides on the next round's pass
            // (two launches per round, every table word read once and written once); `pending`: the tables are still stored at
            // twice r->len
            bool pending = false;
            for (; i < nd && !rc && r->len > r->tail_len; i++) {
                const int eval_one = have_claim ? 0 : 1;
                // While a round's arithmetic fills the machine (the first rounds of a large cube) the fused pass is the slower
                // one (it folds both halves before it can evaluate: measured 79 us against 40 + 15 at 2^19 pairs); once a round
                // is down at the launch floor it saves one launch of three.
                if (pending && r->len / 2 > FUSED_FOLD_MAX_PAIRS) {
                    cudaError_t e = hlk::sc_fold(r->d_tables, r->stride, (u32)r->len, r->k, r->d_state, c->stream);
                    c->stats.kernel_launches++;
                    if (e != cudaSuccess) { rc = fail(c, HL_B200_ERR_DEVICE, "fold launch", e); break; }
                    pending = false;
                }
                if (!pending) {
                    rc = launch_round(r, eval_one, 1, have_claim ? 1 : 0, fs->recover_one ? 1 : 0, d_mask, d_mtab, (int)mask_vars);
                } else {
                    const u32 nb = hlk::sc_round_blocks((u32)(r->len / 2), c->sm_count);
                    cudaError_t e = hlk::sc_fold_round(r->poly, (int)r->k, r->d_tables, r->stride, (u32)r->len, r->d_coefs, r->d_state, eval_one, r->d_partials,
                                                       nb, c->stream);
                    c->stats.kernel_launches++;
                    if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "fold + round launch", e);
                    if (!rc) rc = launch_step(r, nb, 1, have_claim ? 1 : 0, fs->recover_one ? 1 : 0, d_mask, d_mtab, (int)mask_vars);
                }
                r->len /= 2;
                r->next++;
                pending = true;
                have_claim = fs->recover_one != 0;
            }
            if (!rc && pending) {  // the last challenge's fold
                cudaError_t e = hlk::sc_fold(r->d_tables, r->stride, (u32)r->len, r->k, r->d_state, c->stream);
                c->stats.kernel_launches++;
                if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "fold launch", e);
            }
        }
        if (!rc && i < nd) {  // the short rounds: one CTA, no launches in between
            hlk::ScStep a;
            a.partials = r->d_partials; a.nblocks = 1; a.degree = (int)r->degree; a.round = (int)r->next;
            a.use_claim = 0; a.recover = fs->recover_one ? 1 : 0; a.fs = 1; a.mask = d_mask; a.mask_tab = d_mtab; a.mask_vars = (int)mask_vars;
            a.inv_den = r->d_inv_den; a.state = r->d_state; a.out = r->d_out;
            a.eval_degree = (int)r->eval_degree; a.extrap = r->d_extrap;
            const u32 left = nd - i;
            cudaError_t e = r->poly == hlk::POLY_IR
                                ? hlk::sc_tail_ir(r->ir, (int)r->k, r->d_tables, r->stride, (u32)r->len, (int)r->degree, a, (int)left, have_claim ? 1 : 0, c->stream)
                                : hlk::sc_tail(r->poly, (int)r->k, r->d_tables, r->stride, (u32)r->len, r->d_coefs, a, (int)left, have_claim ? 1 : 0,
                                               r->d_partials, c->stream);
            c->stats.kernel_launches++;
            if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "tail rounds launch", e);
            r->len >>= left;
            r->next += left;
        }
    }
    if (!rc) rc = d2h(c, out, r->d_out + (size_t)first * r->out_row(), (size_t)nd * r->out_row() * 8);
    if (!rc) rc = d2h(c, &st, r->d_state, sizeof st);
    if (!rc) rc = sync(c, "rounds_batched");
    if (d_mask) dev_free(c, d_mask, mlen * 16);
    if (d_mtab) dev_free(c, d_mtab, tab_words * 8);
    if (rc) return rc;
    memcpy(fs->state, st.state, 32);
    fs->counter = st.counter;
    fs->claim[0] = st.claim.c0; fs->claim[1] = st.claim.c1;
    fs->have_claim = fs->recover_one ? 1 : fs->have_claim;
    c->stats.round_batches++;
    return HL_B200_OK;
}

}  // extern "C"
