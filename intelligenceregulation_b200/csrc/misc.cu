// Small kernels: the field self-test.
#include "gl_field.cuh"
#include "kernels.h"

namespace {
// (a + b, a - b, a * b) per pair: the device-arithmetic gate every other kernel rests on
__global__ void k_probe_field(const u64* __restrict__ a, const u64* __restrict__ b, size_t n, u64* __restrict__ out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    u64 x = a[i], y = b[i];
    out[3 * i] = gl_add(x, y);
    out[3 * i + 1] = gl_sub(x, y);
    out[3 * i + 2] = gl_mul(x, y);
}
}  // namespace

namespace hlk {
cudaError_t probe_field(const u64* d_a, const u64* d_b, size_t n, u64* d_out3, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    k_probe_field<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(d_a, d_b, n, d_out3);
    return cudaGetLastError();
}
}  // namespace hlk
