/* CPU restatement of the witness weight product, test infrastructure only.
 * hashline/src/private_block/witness.rs:979-991 (matmul_reference): out[t * os + j] = sum_i x[t * xs + i] * w(i, j),
 * w(i, j) = w[j * inner + i], or w[i * outer + j] when in_out; the rest of the out_len plane zero.  Integer arithmetic in
 * int64, so any summation order gives the reference's words. */
#include <stdint.h>
#include <string.h>
#include <stddef.h>

void or_witness_product(size_t t_rows, const int64_t *x, size_t xs, const int8_t *w, size_t inner, size_t outer, size_t os, size_t out_len,
                        int in_out, int64_t *out) {
    memset(out, 0, out_len * sizeof(int64_t));
#pragma omp parallel for collapse(2) schedule(static)
    for (size_t t = 0; t < t_rows; t++)
        for (size_t j = 0; j < outer; j++) {
            int64_t acc = 0;
            if (in_out)
                for (size_t i = 0; i < inner; i++) acc += x[t * xs + i] * (int64_t)w[i * outer + j];
            else
                for (size_t i = 0; i < inner; i++) acc += x[t * xs + i] * (int64_t)w[j * inner + i];
            out[t * os + j] = acc;
        }
}
