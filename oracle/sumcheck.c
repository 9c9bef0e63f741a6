/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * CPU restatement of the reference's multilinear helpers (zkp-core/src/mle.rs),
 * sumcheck rounds / folds (sumcheck.rs:52-136, sumcheck/rounds.rs:33-167) and the
 * CFS masking polynomial (sumcheck.rs:194-319).
 *
 * Tables are k contiguous arrays of `stride` Fp2 (two u64 each); the live part of
 * a table is its first `len` entries.  Variable 0 is the most significant index
 * bit: a round pairs entry i with entry i + len/2.
 */
#include "hl_oracle.h"
#include <stdlib.h>
#include <string.h>

static inline fp2_t ld2(const uint64_t *p) { return fp2_new(p[0], p[1]); }
static inline void st2(uint64_t *p, fp2_t v) { p[0] = v.c0; p[1] = v.c1; }
static inline fp2_t fp2_from_u64(uint64_t v) { return fp2_new(fp_new(v), 0); }

/* mle.rs:17-51: each r splits every entry e into (e(1-r), e r); the FIRST r ends
 * up as the least significant index bit */
void or_eq_table(const uint64_t *r, size_t n, uint64_t *out) {
    fp2_t *o = (fp2_t *)out;
    o[0] = FP2_ONE;
    size_t len = 1;
    for (size_t v = 0; v < n; v++) {
        fp2_t ri = ld2(r + 2 * v), om = fp2_sub(FP2_ONE, ri);
        for (size_t a = 0; a < len; a++) {
            fp2_t e = o[a];
            o[a + len] = fp2_mul(e, ri);
            o[a] = fp2_mul(e, om);
        }
        len <<= 1;
    }
}
/* mle.rs:56-59: r[0] the most significant bit */
void or_eq_table_msb(const uint64_t *r, size_t n, uint64_t *out) {
    uint64_t *rev = (uint64_t *)malloc((n ? n : 1) * 16);
    for (size_t i = 0; i < n; i++) { rev[2 * i] = r[2 * (n - 1 - i)]; rev[2 * i + 1] = r[2 * (n - 1 - i) + 1]; }
    or_eq_table(rev, n, out);
    free(rev);
}

/* mle.rs:338-351: Lagrange through the points 0..d-1 */
static fp2_t interp(const fp2_t *vals, size_t d, fp2_t x) {
    fp2_t acc = FP2_ZERO;
    for (size_t i = 0; i < d; i++) {
        fp2_t num = FP2_ONE;
        uint64_t den = 1;
        for (size_t j = 0; j < d; j++) {
            if (i == j) continue;
            num = fp2_mul(num, fp2_new(fp_sub(x.c0, fp_new(j)), x.c1));
            den = fp_mul(den, fp_from_i64((int64_t)i - (int64_t)j));
        }
        acc = fp2_add(acc, fp2_mul_base(fp2_mul(vals[i], num), fp_inv(den)));
    }
    return acc;
}
void or_interpolate_eval(const uint64_t *vals, size_t d, const uint64_t x[2], uint64_t out[2]) {
    st2(out, interp((const fp2_t *)vals, d, ld2(x)));
}

/* mle.rs:157-185 (fold_rows_i8): out[j] = sum_i w[i] * M[i][j]; the deferred
 * integer form (mle.rs:256-295) gives the same field elements */
void or_fold_rows_i8(const int8_t *m, size_t rows, size_t cols, const uint64_t *w, uint64_t *out) {
#pragma omp parallel for
    for (size_t j = 0; j < cols; j++) {
        fp2_t acc = FP2_ZERO;
        for (size_t i = 0; i < rows; i++) {
            int v = m[i * cols + j];
            if (v) acc = fp2_add(acc, fp2_mul_base(ld2(w + 2 * i), fp_from_i64(v)));
        }
        st2(out + 2 * j, acc);
    }
}
/* mle.rs:187-205 (fold_cols_i8): out[i] = sum_j c[j] * M[i][j] */
void or_fold_cols_i8(const int8_t *m, size_t rows, size_t cols, const uint64_t *c, uint64_t *out) {
#pragma omp parallel for
    for (size_t i = 0; i < rows; i++) {
        fp2_t acc = FP2_ZERO;
        for (size_t j = 0; j < cols; j++) {
            int v = m[i * cols + j];
            if (v) acc = fp2_add(acc, fp2_mul_base(ld2(c + 2 * j), fp_from_i64(v)));
        }
        st2(out + 2 * i, acc);
    }
}

/* ---- poly id 4: a slot polynomial given as data ------------------------------------------------
 * The interpreter of private_block/slot_ir.rs:352-377 (`SlotIr::eval`): nodes in order, an affine node
 * folds konst + sum coef * table (:356), a sum node folds coef * prod(factors) per subterm (:357-360),
 * the value is the sum over terms of coef * prod(wrapper) * prod(inner) (:365-375).  The graph arrives
 * as the 32-bit word stream documented in include/hl_b200.h; or_ir_set keeps the caller's pointer. */
static struct { const uint32_t *w; size_t n_nodes, n_terms; } g_ir;
void or_ir_set(const uint32_t *words, size_t n_nodes, size_t n_terms) {
    g_ir.w = words; g_ir.n_nodes = n_nodes; g_ir.n_terms = n_terms;
}
static fp2_t ir_coef(uint32_t ci, const fp2_t *coefs) {
    if (ci == 0xFFFFFFFFu) return FP2_ONE;
    if (ci == 0xFFFFFFFEu) return fp2_sub(FP2_ZERO, FP2_ONE);
    if (ci == 0xFFFFFFFDu) return FP2_ZERO;
    return coefs[ci];
}
static fp2_t ir_product(const uint32_t **pw, const fp2_t *coefs, const fp2_t *v, const fp2_t *nv) {
    const uint32_t *w = *pw;
    fp2_t p = ir_coef(w[0], coefs);
    uint32_t nf = w[1];
    w += 2;
    for (uint32_t i = 0; i < nf; i++, w++) p = fp2_mul(p, (*w & 0x80000000u) ? nv[*w & 0x7FFFFFFFu] : v[*w]);
    *pw = w;
    return p;
}
static fp2_t ir_eval(const fp2_t *v, const fp2_t *coefs) {
    fp2_t nv[128];
    const uint32_t *w = g_ir.w;
    for (size_t n = 0; n < g_ir.n_nodes; n++) {
        uint32_t head = *w++, cnt = head >> 8;
        fp2_t a;
        if ((head & 0xFF) == 0) {
            a = ir_coef(*w++, coefs);
            for (uint32_t i = 0; i < cnt; i++, w += 2) a = fp2_add(a, fp2_mul(ir_coef(w[0], coefs), v[w[1]]));
        } else {
            a = FP2_ZERO;
            for (uint32_t i = 0; i < cnt; i++) a = fp2_add(a, ir_product(&w, coefs, v, nv));
        }
        nv[n] = a;
    }
    fp2_t total = FP2_ZERO;
    for (size_t t = 0; t < g_ir.n_terms; t++) total = fp2_add(total, ir_product(&w, coefs, v, nv));
    return total;
}

static fp2_t poly_eval(int poly, const fp2_t *v, size_t k, const fp2_t *coefs) {
    switch (poly) {
    case 4: return ir_eval(v, coefs);
    case 0: { /* the "prod" family of the L6 corpus; slot matmuls v0*v1 (argument.rs:2174-2203) */
        fp2_t a = FP2_ONE;
        for (size_t t = 0; t < k; t++) a = fp2_mul(a, v[t]);
        return a;
    }
    case 1: /* the "zc" family of the L6 corpus: eq * (a*b - c) */
        return fp2_mul(v[0], fp2_sub(fp2_mul(v[1], v[2]), v[3]));
    case 2: /* LogUp query side: eq * (h * (alpha - q) - 1) */
        return fp2_mul(v[0], fp2_sub(fp2_mul(v[1], fp2_sub(coefs[0], v[2])), FP2_ONE));
    case 3: /* LogUp table side: eq * (h_t * (alpha - t) - m) (layout.rs slot 19) */
        return fp2_mul(v[0], fp2_sub(fp2_mul(v[1], fp2_sub(coefs[0], v[2])), v[3]));
    }
    return FP2_ZERO;
}
void or_poly_eval(int poly, const uint64_t *vals, size_t k, const uint64_t *coefs, uint64_t out[2]) {
    st2(out, poly_eval(poly, (const fp2_t *)vals, k, (const fp2_t *)coefs));
}

/* sumcheck/rounds.rs:94-136: values at 0..=degree of sum_i poly(T(i) + d (T(i+half) - T(i)))
 * by repeated addition; with eval_one == 0 the point 1 is skipped (left zero). */
void or_sc_round(int poly, const uint64_t *tables, size_t k, size_t len, size_t degree, const uint64_t *coefs,
                 int eval_one, uint64_t *sums) {
    /* `tables` here is k arrays at stride `len` */
    size_t half = len / 2;
    fp2_t acc[16];
    for (size_t d = 0; d <= degree; d++) acc[d] = FP2_ZERO;
#pragma omp parallel
    {
        fp2_t loc[16], cur[64], dif[64];
        for (size_t d = 0; d <= degree; d++) loc[d] = FP2_ZERO;
#pragma omp for nowait
        for (size_t i = 0; i < half; i++) {
            for (size_t t = 0; t < k; t++) {
                const uint64_t *tb = tables + 2 * t * len;
                cur[t] = ld2(tb + 2 * i);
                dif[t] = fp2_sub(ld2(tb + 2 * (i + half)), cur[t]);
            }
            loc[0] = fp2_add(loc[0], poly_eval(poly, cur, k, (const fp2_t *)coefs));
            for (size_t d = 1; d <= degree; d++) {
                for (size_t t = 0; t < k; t++) cur[t] = fp2_add(cur[t], dif[t]);
                if (d != 1 || eval_one) loc[d] = fp2_add(loc[d], poly_eval(poly, cur, k, (const fp2_t *)coefs));
            }
        }
#pragma omp critical(or_sc_round)
        for (size_t d = 0; d <= degree; d++) acc[d] = fp2_add(acc[d], loc[d]);
    }
    for (size_t d = 0; d <= degree; d++) st2(sums + 2 * d, acc[d]);
}

/* sumcheck/rounds.rs:145-160: T[i] += r (T[i+half] - T[i]) on the first half */
void or_sc_fold(uint64_t *tables, size_t k, size_t len, size_t stride, const uint64_t r[2]) {
    size_t half = len / 2;
    fp2_t rr = ld2(r);
    for (size_t t = 0; t < k; t++) {
        uint64_t *tb = tables + 2 * t * stride;
#pragma omp parallel for if (half >= 4096)
        for (size_t i = 0; i < half; i++) {
            fp2_t a = ld2(tb + 2 * i), b = ld2(tb + 2 * (i + half));
            st2(tb + 2 * i, fp2_add(a, fp2_mul(rr, fp2_sub(b, a))));
        }
    }
}

/* sumcheck.rs:194-279.  Coefficients [a0, a', a_{0,1..d}, a_{1,1..d}, ...]. */
static fp2_t cfs_u(const fp2_t *co, size_t degree, size_t j, fp2_t x) {
    fp2_t acc = FP2_ZERO, xp = FP2_ONE;
    for (size_t e = 1; e <= degree; e++) {
        xp = fp2_mul(xp, x);
        acc = fp2_add(acc, fp2_mul(co[2 + j * degree + (e - 1)], xp));
    }
    return acc;
}
void or_cfs_round(const uint64_t *coeffs, size_t n_vars, size_t degree, size_t j, const uint64_t *prev, uint64_t *out) {
    const fp2_t *co = (const fp2_t *)coeffs;
    uint64_t half = fp_inv(2);
    fp2_t base = co[0], prod = FP2_ONE;
    for (size_t i = 0; i < j; i++) base = fp2_add(base, cfs_u(co, degree, i, ld2(prev + 2 * i)));
    for (size_t i = j + 1; i < n_vars; i++) base = fp2_add(base, fp2_mul_base(cfs_u(co, degree, i, FP2_ONE), half));
    fp2_t scale = fp2_from_u64((uint64_t)1 << (n_vars - 1 - j));
    for (size_t i = 0; i < j; i++) prod = fp2_mul(prod, ld2(prev + 2 * i));
    for (size_t x = 0; x <= degree; x++) {
        fp2_t xv = fp2_from_u64(x);
        fp2_t v = fp2_add(fp2_mul(scale, fp2_add(base, cfs_u(co, degree, j, xv))), fp2_mul(fp2_mul(co[1], prod), xv));
        st2(out + 2 * x, v);
    }
}
void or_cfs_total(const uint64_t *coeffs, size_t n_vars, size_t degree, uint64_t out[2]) {
    const fp2_t *co = (const fp2_t *)coeffs;
    size_t len = n_vars * degree + 2;
    fp2_t acc = FP2_ZERO;
    for (size_t i = 0; i < len; i++) {
        fp2_t w = i == 0 ? fp2_from_u64((uint64_t)1 << n_vars) : i == 1 ? FP2_ONE : fp2_from_u64((uint64_t)1 << (n_vars - 1));
        acc = fp2_add(acc, fp2_mul(w, co[i]));
    }
    st2(out, acc);
}
void or_cfs_eval(const uint64_t *coeffs, size_t n_vars, size_t degree, const uint64_t *rho, uint64_t out[2]) {
    const fp2_t *co = (const fp2_t *)coeffs;
    fp2_t prod = FP2_ONE, acc = co[0];
    for (size_t i = 0; i < n_vars; i++) prod = fp2_mul(prod, ld2(rho + 2 * i));
    acc = fp2_add(acc, fp2_mul(prod, co[1]));
    size_t at = 2;
    for (size_t i = 0; i < n_vars; i++) {
        fp2_t xp = FP2_ONE;
        for (size_t e = 0; e < degree; e++) {
            xp = fp2_mul(xp, ld2(rho + 2 * i));
            acc = fp2_add(acc, fp2_mul(xp, co[at++]));
        }
    }
    st2(out, acc);
}

/* The driver of sumcheck/rounds.rs:33-48 with the transcript masker of
 * sumcheck.rs:282-299 / transcript.rs:89-100 folded in, and the s(1) recovery of
 * sumcheck/rounds.rs:94-147. */
void or_sc_prove(int poly, uint64_t *tables, size_t k, size_t n_vars, size_t degree, const uint64_t *coefs,
                 const uint64_t *mask, const uint64_t mask_c[2], size_t mask_vars, int recover_one,
                 const uint64_t *claim, or_transcript *tr,
                 uint64_t *out_rounds, uint64_t *out_masked, uint64_t *out_chal, uint64_t *out_finals) {
    size_t stride = (size_t)1 << n_vars, len = stride, w = degree + 1;
    int have_claim = recover_one && claim != NULL;
    fp2_t cl = have_claim ? ld2(claim) : FP2_ZERO;
    uint64_t *packed = (uint64_t *)malloc(2 * k * stride * 8);
    for (size_t j = 0; j < n_vars; j++) {
        uint64_t *sums = out_rounds + 2 * w * j, *msg = out_masked + 2 * w * j;
        /* or_sc_round wants the live halves packed at stride len */
        for (size_t t = 0; t < k; t++) memcpy(packed + 2 * t * len, tables + 2 * t * stride, len * 16);
        or_sc_round(poly, packed, k, len, degree, coefs, !have_claim, sums);
        if (have_claim) st2(sums + 2, fp2_sub(cl, ld2(sums)));
        memcpy(msg, sums, w * 16);
        if (mask) {
            uint64_t g[2 * 16];
            or_cfs_round(mask, mask_vars, degree, j, out_chal, g);
            for (size_t d = 0; d < w; d++) st2(msg + 2 * d, fp2_add(ld2(sums + 2 * d), fp2_mul(ld2(mask_c), ld2(g + 2 * d))));
        }
        or_tr_absorb(tr, (const uint8_t *)"sc-round", 8, (const uint8_t *)msg, w * 16);
        or_tr_challenge_fp2(tr, out_chal + 2 * j);
        if (recover_one) { cl = interp((const fp2_t *)sums, w, ld2(out_chal + 2 * j)); have_claim = 1; }
        or_sc_fold(tables, k, len, stride, out_chal + 2 * j);
        len /= 2;
    }
    free(packed);
    for (size_t t = 0; t < k; t++) { out_finals[2 * t] = tables[2 * t * stride]; out_finals[2 * t + 1] = tables[2 * t * stride + 1]; }
}
