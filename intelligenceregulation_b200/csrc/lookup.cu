// LogUp helper columns of table-indexed lookups (hashline/src/private_block/protocol.rs:1125-1230, 1700-1800): the byte
// tables and the 16-bit range families, ~32 M looked words per 8B block.
//
// The denominators alpha - (v + g) take only 2^w values, so the reference inverts a TABLE once (u8_denominator_inverses:
// the non-zero denominators in one Montgomery batch, a zero one marked absent) and every looked word reads its entry;
// a paired job writes the sum of two columns' entries; a word outside the table (only a tampered witness carries one)
// takes the direct inversion; a word whose denominator is zero refuses the attempt ("zero LogUp denominator", never
// resampled).  A zero denominator at a value NO word carries does not refuse here (protocol.rs:1142-1162).
//
//   k_inverse_table  entry v = 1 / (alpha - (v + g)), or (0, 0) where the denominator is zero (an inverse is never zero)
//   k_lookup_helpers re[i], im[i] = entry(a[i]) (+ entry(b[i])), the two planes of H the reference writes
#include "api_internal.h"
#include "gl_field.cuh"

using namespace hlapi;

namespace {

constexpr int TB = 8;  // table entries per thread: one inversion per TB entries

__global__ void __launch_bounds__(128) k_inverse_table(fp2 alpha_minus_g, u32 len, u64* __restrict__ table) {
    const u32 v0 = (blockIdx.x * blockDim.x + threadIdx.x) * TB;
    if (v0 >= len) return;
    fp2 d[TB], pre[TB];
    fp2 acc = f2(1, 0);
#pragma unroll
    for (int j = 0; j < TB; j++) {
        d[j] = v0 + j < len ? f2(gl_sub(alpha_minus_g.c0, (u64)(v0 + j)), alpha_minus_g.c1) : f2(1, 0);
        pre[j] = acc;
        if (!f2_is_zero(d[j])) acc = f2_mul(acc, d[j]);  // a zero denominator stays out of the batch
    }
    fp2 inv = f2_inv(acc);
#pragma unroll
    for (int j = TB - 1; j >= 0; j--) {
        fp2 r = f2(0, 0);
        if (!f2_is_zero(d[j])) {
            r = f2_mul(inv, pre[j]);
            inv = f2_mul(inv, d[j]);
        }
        if (v0 + j < len) *reinterpret_cast<ulonglong2*>(table + 2 * (size_t)(v0 + j)) = make_ulonglong2(r.c0, r.c1);
    }
}

struct Col {
    const long long* v;   // looked words
    const u64* table;     // 2^log_len entries
    u32 len;
    fp2 alpha_minus_g;
};

// helper_one_any (protocol.rs:1168-1182): the table entry for a word inside the table, the direct inverse otherwise
__device__ __forceinline__ bool helper_one(const Col& c, size_t i, fp2& out) {
    const long long v = c.v[i];
    if (v >= 0 && (unsigned long long)v < c.len) {
        const ulonglong2 e = *reinterpret_cast<const ulonglong2*>(c.table + 2 * (size_t)v);
        out = f2(e.x, e.y);
        return (e.x | e.y) != 0;
    }
    const fp2 d = f2(gl_sub(c.alpha_minus_g.c0, gl_from_i64(v)), c.alpha_minus_g.c1);
    if (f2_is_zero(d)) return false;
    out = f2_inv(d);
    return true;
}

// two looked words per thread: 16-byte reads of the columns and 16-byte writes of the planes where the addresses allow
__global__ void __launch_bounds__(256) k_lookup_helpers(Col a, Col b, int paired, size_t n, u64* __restrict__ re, u64* __restrict__ im,
                                                        int* __restrict__ err) {
    const size_t i0 = 2 * ((size_t)blockIdx.x * blockDim.x + threadIdx.x);
    if (i0 >= n) return;
    const int cnt = i0 + 1 < n ? 2 : 1;
    u64 r[2] = {0, 0}, m[2] = {0, 0};
    bool ok = true;
#pragma unroll
    for (int e = 0; e < 2; e++) {
        if (e < cnt) {
            fp2 h, y;
            bool good = helper_one(a, i0 + e, h);
            if (good && paired) {
                good = helper_one(b, i0 + e, y);
                if (good) h = f2_add(h, y);
            }
            ok &= good;
            r[e] = h.c0;
            m[e] = h.c1;
        }
    }
    if (!ok) { atomicExch(err, 1); return; }
    const bool wide = cnt == 2 && ((reinterpret_cast<uintptr_t>(re + i0) | reinterpret_cast<uintptr_t>(im + i0)) & 15) == 0;
    if (wide) {
        *reinterpret_cast<ulonglong2*>(re + i0) = make_ulonglong2(r[0], r[1]);
        *reinterpret_cast<ulonglong2*>(im + i0) = make_ulonglong2(m[0], m[1]);
    } else {
        for (int e = 0; e < cnt; e++) { re[i0 + e] = r[e]; im[i0 + e] = m[e]; }
    }
}

int check_log(hl_ctx* c, uint32_t log_len) {
    return log_len > 24 ? fail(c, HL_B200_ERR_UNSUPPORTED, "lookup: table above 2^24 entries") : HL_B200_OK;
}

}  // namespace

extern "C" {

int hl_b200_lookup_inverse_table(hl_ctx* c, const uint64_t alpha[2], const uint64_t g[2], uint32_t log_len, uint64_t* d_table) {
    if (!c || !alpha || !g || !d_table) return fail(c, HL_B200_ERR_ARG, "lookup_inverse_table: null argument");
    if (int rc = check_log(c, log_len)) return rc;
    if ((uintptr_t)d_table & 15) return fail(c, HL_B200_ERR_ARG, "lookup_inverse_table: the table must be 16-byte aligned");
    std::lock_guard<std::mutex> lk(c->mu);
    cudaSetDevice(c->device);
    const u32 len = 1u << log_len;
    const fp2 amg = f2_sub(f2(alpha[0], alpha[1]), f2(g[0], g[1]));
    Timed t(c, HL_T_LOGUP);
    k_inverse_table<<<(len / TB + 127) / 128 + 1, 128, 0, c->stream>>>(amg, len, reinterpret_cast<u64*>(d_table));
    c->stats.kernel_launches++;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? HL_B200_OK : fail(c, HL_B200_ERR_DEVICE, "inverse table launch", e);
}

int hl_b200_lookup_helpers_dev(hl_ctx* c, const int64_t* d_a, const uint64_t* d_table_a, uint32_t log_a, const uint64_t g_a[2],
                               const int64_t* d_b, const uint64_t* d_table_b, uint32_t log_b, const uint64_t g_b[2],
                               const uint64_t alpha[2], size_t n, uint64_t* d_re, uint64_t* d_im) {
    if (!c || !d_a || !d_table_a || !g_a || !alpha || (n && (!d_re || !d_im))) return fail(c, HL_B200_ERR_ARG, "lookup_helpers: null argument");
    if (d_b && (!d_table_b || !g_b)) return fail(c, HL_B200_ERR_ARG, "lookup_helpers: the second column needs its table and tag");
    if (int rc = check_log(c, log_a)) return rc;
    if (d_b) if (int rc = check_log(c, log_b)) return rc;
    if (n == 0) return HL_B200_OK;
    if (((uintptr_t)d_table_a & 15) || ((uintptr_t)d_table_b & 15) || ((uintptr_t)d_a & 7) || ((uintptr_t)d_b & 7) || ((uintptr_t)d_re & 7) || ((uintptr_t)d_im & 7))
        return fail(c, HL_B200_ERR_ARG, "lookup_helpers: tables must be 16-byte aligned, columns and planes 8-byte aligned");
    std::lock_guard<std::mutex> lk(c->mu);
    cudaSetDevice(c->device);
    int* d_err = nullptr;
    int rc = dev_alloc(c, (void**)&d_err, 4);
    if (!rc && cudaMemsetAsync(d_err, 0, 4, c->stream) != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "lookup_helpers: flag");
    const fp2 al = f2(alpha[0], alpha[1]);
    Col a{reinterpret_cast<const long long*>(d_a), reinterpret_cast<const u64*>(d_table_a), 1u << log_a, f2_sub(al, f2(g_a[0], g_a[1]))};
    Col b = a;
    if (d_b) b = Col{reinterpret_cast<const long long*>(d_b), reinterpret_cast<const u64*>(d_table_b), 1u << log_b, f2_sub(al, f2(g_b[0], g_b[1]))};
    if (!rc) {
        Timed t(c, HL_T_LOGUP);
        k_lookup_helpers<<<(unsigned)((n + 511) / 512), 256, 0, c->stream>>>(a, b, d_b ? 1 : 0, n, reinterpret_cast<u64*>(d_re),
                                                                            reinterpret_cast<u64*>(d_im), d_err);
        c->stats.kernel_launches++;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "lookup helpers launch", e);
    }
    int flag = 0;
    if (!rc) rc = d2h(c, &flag, d_err, 4);
    if (!rc) rc = sync(c, "lookup_helpers");
    if (d_err) dev_free(c, d_err, 4);
    if (!rc && flag) rc = fail(c, HL_B200_ERR_ZERO, "zero LogUp denominator; discard attempt");
    return rc;
}

}  // extern "C"
