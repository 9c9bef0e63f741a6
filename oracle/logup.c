/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * CPU restatement of the reference's LogUp helper arithmetic
 * (hashline/src/private_block/protocol.rs:993-1011 `inverses`, :1928-1933
 * `table_helper`; accuracy_act.rs:55-117 `histogram`, `query_values`,
 * `denominators`) for a single-group lookup of (index, output) pairs:
 *
 *   query tuple   q_i = (idx_i + idx_off) + beta * out_i + tag
 *   helper        h_i = 1 / (alpha - q_i)
 *   table tuple   t_v = v + beta * table_out[v] + tag        (v = 0 .. table_len-1)
 *   table helper  h_t[v] = mult[v] / (alpha - t_v)
 *
 * All sums are formed in the field (Fp2::from_i64 of each term), never through
 * wrapping signed arithmetic, as accuracy_act.rs:91-99 requires.
 */
#include "hl_oracle.h"
#include <stdlib.h>
#include <string.h>

static inline fp2_t from_i64(int64_t v) { return fp2_new(fp_from_i64(v), 0); }

/* accuracy_act.rs:55-73: every query counted (padding included) */
void or_logup_histogram(const int32_t *idx, size_t nq, size_t table_len, uint64_t *mult) {
    memset(mult, 0, table_len * 8);
    for (size_t i = 0; i < nq; i++) mult[(size_t)idx[i]]++;
}

/* protocol.rs:993-1011: denominators inverted in chunks of 2^14 by Montgomery's
 * trick (field.rs:212-227); inverses are unique, so chunking moves no word. */
void or_logup_helpers(const int32_t *idx, const int32_t *outv, size_t nq, const uint64_t alpha[2],
                      const uint64_t beta[2], const uint64_t gamma_tag[2], int64_t idx_off, uint64_t *h) {
    fp2_t a = fp2_new(alpha[0], alpha[1]), b = fp2_new(beta[0], beta[1]), tag = fp2_new(gamma_tag[0], gamma_tag[1]);
    fp2_t *den = (fp2_t *)h;
    const size_t CH = (size_t)1 << 14;
    size_t nch = (nq + CH - 1) / CH;
#pragma omp parallel for schedule(dynamic, 1)
    for (size_t c = 0; c < nch; c++) {
        size_t lo = c * CH, hi = lo + CH < nq ? lo + CH : nq;
        for (size_t i = lo; i < hi; i++) {
            fp2_t q = fp2_add(fp2_add(fp2_add(from_i64(idx[i]), from_i64(idx_off)), fp2_mul(b, from_i64(outv[i]))), tag);
            den[i] = fp2_sub(a, q);
        }
        or_batch_inverse2((uint64_t *)(den + lo), hi - lo);
    }
}

/* protocol.rs:1928-1933 with the table tuple of accuracy_act.rs:28-31 */
void or_logup_table_helper(const int32_t *table_out, const uint64_t *mult, size_t table_len, const uint64_t alpha[2],
                           const uint64_t beta[2], const uint64_t gamma_tag[2], uint64_t *ht) {
    fp2_t a = fp2_new(alpha[0], alpha[1]), b = fp2_new(beta[0], beta[1]), tag = fp2_new(gamma_tag[0], gamma_tag[1]);
    fp2_t *den = (fp2_t *)ht;
    for (size_t v = 0; v < table_len; v++) {
        fp2_t t = fp2_add(fp2_add(from_i64((int64_t)v), fp2_mul(b, from_i64(table_out[v]))), tag);
        den[v] = fp2_sub(a, t);
    }
    or_batch_inverse2(ht, table_len);
    for (size_t v = 0; v < table_len; v++) den[v] = fp2_mul_base(den[v], fp_new(mult[v]));
}

/* accuracy_act.rs:91-99 (query_values): q_i = (idx_i + off) + beta * out_i + tag; idx NULL means idx_i = i */
void or_logup_query_values(const int32_t *idx, const int32_t *outv, size_t n, const uint64_t beta[2],
                           const uint64_t gamma_tag[2], int64_t idx_off, uint64_t *q) {
    fp2_t b = fp2_new(beta[0], beta[1]), tag = fp2_new(gamma_tag[0], gamma_tag[1]);
    fp2_t *o = (fp2_t *)q;
#pragma omp parallel for
    for (size_t i = 0; i < n; i++) {
        int64_t a = idx ? (int64_t)idx[i] : (int64_t)i;
        o[i] = fp2_add(fp2_add(fp2_add(from_i64(a), from_i64(idx_off)), fp2_mul(b, from_i64(outv[i]))), tag);
    }
}

/* sum of an Fp2 vector */
void or_fp2_sum(const uint64_t *v, size_t n, uint64_t out[2]) {
    fp2_t acc = FP2_ZERO;
    for (size_t i = 0; i < n; i++) acc = fp2_add(acc, fp2_new(v[2 * i], v[2 * i + 1]));
    out[0] = acc.c0; out[1] = acc.c1;
}

/* protocol.rs:1125-1140 (u8_denominator_inverses): table[v] = 1/(alpha - (v + g)), the non-zero denominators in one
 * batch inversion; absent[v] = 1 where the denominator is zero (the entry is then left (0, 0)). */
void or_lookup_inverse_table(const uint64_t alpha[2], const uint64_t g[2], size_t len, uint64_t *table, uint8_t *absent) {
    fp2_t a = fp2_new(alpha[0], alpha[1]), gg = fp2_new(g[0], g[1]);
    fp2_t *nz = (fp2_t *)malloc(sizeof(fp2_t) * (len ? len : 1));
    size_t k = 0;
    for (size_t v = 0; v < len; v++) {
        fp2_t d = fp2_sub(a, fp2_add(from_i64((int64_t)v), gg));
        absent[v] = (d.c0 | d.c1) == 0;
        if (!absent[v]) nz[k++] = d;
    }
    or_batch_inverse2((uint64_t *)nz, k);
    k = 0;
    for (size_t v = 0; v < len; v++) {
        fp2_t e = absent[v] ? fp2_new(0, 0) : nz[k++];
        table[2 * v] = e.c0;
        table[2 * v + 1] = e.c1;
    }
    free(nz);
}

/* protocol.rs:1168-1182 (helper_one) */
static int lookup_one(int64_t v, fp2_t a, fp2_t g, const uint64_t *table, const uint8_t *absent, size_t len, fp2_t *out) {
    if (v >= 0 && (uint64_t)v < len) {
        if (absent[v]) return 0;
        *out = fp2_new(table[2 * v], table[2 * v + 1]);
        return 1;
    }
    fp2_t d = fp2_sub(a, fp2_add(from_i64(v), g));
    if ((d.c0 | d.c1) == 0) return 0;
    *out = fp2_inv(d);
    return 1;
}

/* protocol.rs:1186-1193, 1206-1216 (helper_inverses_u8 / helper_pair_inverses_u8) written as the two planes of H
 * (write_helpers_w16_cols :1730): returns 0, or 1 for "zero LogUp denominator" (the first column asked first). */
int or_lookup_helpers(const int64_t *a, const uint64_t *table_a, const uint8_t *absent_a, size_t len_a, const uint64_t g_a[2],
                      const int64_t *b, const uint64_t *table_b, const uint8_t *absent_b, size_t len_b, const uint64_t g_b[2],
                      const uint64_t alpha[2], size_t n, uint64_t *re, uint64_t *im) {
    fp2_t al = fp2_new(alpha[0], alpha[1]), ga = fp2_new(g_a[0], g_a[1]), gb = b ? fp2_new(g_b[0], g_b[1]) : ga;
    int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
    for (size_t i = 0; i < n; i++) {
        fp2_t h, y;
        if (!lookup_one(a[i], al, ga, table_a, absent_a, len_a, &h)) { bad |= 1; continue; }
        if (b) {
            if (!lookup_one(b[i], al, gb, table_b, absent_b, len_b, &y)) { bad |= 1; continue; }
            h = fp2_add(h, y);
        }
        re[i] = h.c0;
        im[i] = h.c1;
    }
    return bad;
}

/* ---- the three-coordinate activation lookup (private_block/accuracy_act.rs) ---- */
static size_t act_group(size_t index, size_t f_pad, size_t tokens, size_t hidden, const uint32_t *group_ids) {
    /* accuracy_act.rs:52-54 (query_group) */
    return (index / f_pad < tokens && index % f_pad < hidden) ? group_ids[index % f_pad] : 0;
}

/* accuracy_act.rs:61-79 (histogram): returns the misses */
uint64_t or_act_histogram(const int64_t *gates, const int64_t *outputs, size_t n, size_t f_pad, size_t tokens, size_t hidden,
                          const uint32_t *group_ids, const int64_t *tables, size_t groups, uint64_t *counts) {
    uint64_t misses = 0;
    memset(counts, 0, groups * 4096 * sizeof(uint64_t));
    for (size_t i = 0; i < n; i++) {
        size_t group = act_group(i, f_pad, tokens, hidden, group_ids), bucket = 0;
        int64_t g = gates[i];
        int hit = 0;
        if (g >= -2048 && g < 2048) {
            size_t key = (size_t)(g + 2048);
            if (tables[group * 4096 + key] == outputs[i]) { hit = 1; bucket = group * 4096 + key; }
        }
        if (!hit) misses++;
        counts[bucket]++;
    }
    return misses;
}

/* accuracy_act.rs:88-95 (query_values) */
void or_act_query_values(const int64_t *gates, const int64_t *outputs, size_t n, size_t f_pad, size_t tokens, size_t hidden,
                         const uint32_t *group_ids, const uint64_t beta[2], const uint64_t tag[2], uint64_t *q) {
    fp2_t b = fp2_new(beta[0], beta[1]), tg = fp2_new(tag[0], tag[1]), b2 = fp2_mul(b, b);
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        fp2_t v = fp2_add(from_i64(gates[i]), from_i64(2048));
        v = fp2_add(v, fp2_mul(b, from_i64(outputs[i])));
        v = fp2_add(v, fp2_mul(b2, from_i64((int64_t)act_group(i, f_pad, tokens, hidden, group_ids))));
        v = fp2_add(v, tg);
        q[2 * i] = v.c0;
        q[2 * i + 1] = v.c1;
    }
}

/* accuracy_act.rs:13-31 (table): compressed and support, len entries */
void or_act_table(const int64_t *tables, size_t groups, size_t len, const uint64_t beta[2], const uint64_t tag[2], uint64_t *compressed,
                  uint64_t *support) {
    fp2_t b = fp2_new(beta[0], beta[1]), tg = fp2_new(tag[0], tag[1]), b2 = fp2_mul(b, b);
    fp2_t zero = fp2_add(from_i64(2048), tg);
    for (size_t i = 0; i < len; i++) {
        compressed[2 * i] = zero.c0; compressed[2 * i + 1] = zero.c1;
        support[2 * i] = 0; support[2 * i + 1] = 0;
    }
    for (size_t g = 0; g < groups; g++) {
        fp2_t gt = fp2_mul(b2, from_i64((int64_t)g));
        for (size_t k = 0; k < 4096; k++) {
            size_t i = g * 4096 + k;
            fp2_t v = fp2_add(fp2_add(fp2_add(from_i64((int64_t)k), fp2_mul(b, from_i64(tables[i]))), gt), tg);
            compressed[2 * i] = v.c0; compressed[2 * i + 1] = v.c1;
            support[2 * i] = 1;
        }
    }
}
