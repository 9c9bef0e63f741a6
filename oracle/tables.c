/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * CPU restatement of the reference's host table builders for a slot's sumcheck
 * (hashline/src/private_block/argument.rs): the eq cube and the committed-plane table,
 * both in their plain definitional ("walked") form.
 */
#include "hl_oracle.h"
#include <stdlib.h>
#include <string.h>

static inline fp2_t ld2(const uint64_t *p) { return fp2_new(p[0], p[1]); }
static inline void st2(uint64_t *p, fp2_t v) { p[0] = v.c0; p[1] = v.c1; }

/* argument.rs:586-627 eq_cube over eq_table_msb(point): entry x is e[(x >> shift) & (|e| - 1)],
 * shift = n_vars - start - |point| */
void or_eq_cube(const uint64_t *point, size_t p, size_t n_vars, size_t start, uint64_t *out) {
    size_t len = (size_t)1 << n_vars, shift = n_vars - start - p, m = ((size_t)1 << p) - 1;
    uint64_t *e = (uint64_t *)malloc(((size_t)2 << p) * 8);
    or_eq_table_msb(point, p, e);
    for (size_t x = 0; x < len; x++) memcpy(out + 2 * x, e + 2 * ((x >> shift) & m), 16);
    free(e);
}

/* argument.rs:386-398 and 546-577 priv_table_fill, the loop form: coordinate j of the plane reads bit
 * log - 1 - j of the plane index; Rho(k) sends it to cube bit n_vars - 1 - k, Flip(k) its complement,
 * Fixed(f) appends it to z (first fixed coordinate = most significant); out[x] += eqf[z] * v(idx),
 * v(idx) = sum_s coef_s * data[off_s + idx]; then the table is broadcast over the variables it does
 * not read.  kind: 0 Rho, 1 Flip, 2 Fixed; `fixed` holds the Fixed values in coordinate order. */
void or_priv_table(const int32_t *kind, const uint32_t *var, const uint64_t *fixed, size_t log,
                   const uint64_t *slices, size_t ns, const uint64_t *data, size_t n_vars, uint64_t *out) {
    size_t nf = 0, used = 0, len = (size_t)1 << n_vars;
    for (size_t j = 0; j < log; j++) {
        if (kind[j] == 2) nf++;
        else used |= (size_t)1 << (n_vars - 1 - var[j]);
    }
    uint64_t *eqf = (uint64_t *)malloc(((size_t)2 << nf) * 8);
    or_eq_table_msb(fixed, nf, eqf);
    memset(out, 0, len * 16);
    for (size_t idx = 0; idx < ((size_t)1 << log); idx++) {
        size_t x = 0, z = 0;
        for (size_t j = 0; j < log; j++) {
            size_t b = (idx >> (log - 1 - j)) & 1;
            if (kind[j] == 0) x |= b << (n_vars - 1 - var[j]);
            else if (kind[j] == 1) x |= (1 - b) << (n_vars - 1 - var[j]);
            else z = (z << 1) | b;
        }
        fp2_t v = FP2_ZERO;
        for (size_t s = 0; s < ns; s++)
            v = fp2_add(v, fp2_mul(ld2(slices + 3 * s + 1), fp2_new(data[slices[3 * s] + idx], 0)));
        st2(out + 2 * x, fp2_add(ld2(out + 2 * x), fp2_mul(ld2(eqf + 2 * z), v)));
    }
    if (used != len - 1)
        for (size_t x = 0; x < len; x++)
            if (x & ~used) memcpy(out + 2 * x, out + 2 * (x & used), 16);
    free(eqf);
}
