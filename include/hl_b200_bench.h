/* hl_b200_bench.h - measurement aids of the benchmark, exported by the same library but NOT part of the backend's interface.
 *
 * Nothing here has a counterpart in the reference and no prover calls it: bench.py uses these to put a measured integer
 * ceiling beside the encoder and the column hash (the kernels are bound by integer issue, for which the machine has no
 * published peak).
 */
#ifndef HL_B200_BENCH_H
#define HL_B200_BENCH_H
#include "hl_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Runs the encoder's butterfly arithmetic on registers only, on every SM, and reports radix-2 Goldilocks
 * butterflies per second: the denominator for the encoder's integer-pipe utilisation. */
int hl_b200_butterfly_peak(hl_ctx* ctx, uint32_t iters, double* butterflies_per_second);
/* the same for the column hash: register-resident BLAKE3 compressions per second, all SMs */
int hl_b200_compress_peak(hl_ctx* ctx, uint32_t iters, double* compressions_per_second);
/* A/B switch of the sumcheck kernels' programmatic dependent launch (process-wide, on by default): with 0 every kernel of a
 * sumcheck is an ordinary stream launch again.  For measuring what the chained launch saves. */
int hl_b200_set_dependent_launch(int on);

#ifdef __cplusplus
}
#endif
#endif
