// The three-coordinate activation lookup of the accuracy lane (hashline/src/private_block/accuracy_act.rs:13-117): queries
// (gate, output, group) against one to four registered 4096-entry tables, compressed as
//   q = gate + 2048 + beta * output + beta^2 * group + tag        (query_values, :88-95; denominators, :106-124)
//   t = key  + beta * word + beta^2 * group + tag                 (table, :13-31; padding entries 2048 + tag)
// with group = group_ids[column] on a live row (row < tokens, column < hidden) and 0 elsewhere (query_group, :52-54).
//   k_act_hist      bucket = group * 4096 + (gate + 2048) when the key is in range and the table's word equals the output,
//                   else bucket 0 and one more miss (histogram, :61-79); 64-bit atomics, integer counts
//   k_act_helpers   1 / (alpha - q_i) or mult_i / (alpha - t_i), Montgomery batches of 8 per thread; any zero denominator
//                   raises the flag ("zero LogUp denominator; discard attempt", protocol.rs:1005-1006)
// Every term is formed in the field (a forged i64 gate never wraps, :82-83).
#include "api_internal.h"
#include "gl_field.cuh"

using namespace hlapi;

namespace {

struct ActShape {
    u32 f_pad, tokens, hidden;
    const u32* group_ids;  // hidden entries
};

__device__ __forceinline__ u32 query_group(const ActShape& s, size_t index) {
    const size_t row = index / s.f_pad;
    const u32 col = (u32)(index % s.f_pad);
    return row < s.tokens && col < s.hidden ? s.group_ids[col] : 0u;
}

__global__ void __launch_bounds__(256) k_act_hist(const long long* __restrict__ gates, const long long* __restrict__ outputs, size_t n, ActShape s,
                                                  const long long* __restrict__ tables, u32 groups, unsigned long long* __restrict__ counts,
                                                  unsigned long long* __restrict__ misses) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const u32 group = query_group(s, i);
    const long long g = gates[i];
    u32 bucket = 0;
    bool hit = false;
    if (g >= -2048 && g < 2048 && group < groups) {  // checked_add(2048) in 0..4096
        const u32 key = (u32)(g + 2048);
        if (tables[(size_t)group * 4096 + key] == outputs[i]) { hit = true; bucket = group * 4096 + key; }
    }
    if (!hit) atomicAdd(misses, 1ull);
    atomicAdd(counts + bucket, 1ull);
}

constexpr int AB = 8;

// mode 0: queries (a = gates, b = outputs); mode 1: table entries (a = NULL: key = i % 4096, b = table words, group = i / 4096,
// entries from `entries` on are the padding value 2048 + tag), scaled by mult
__global__ void __launch_bounds__(128) k_act_helpers(int mode, const long long* __restrict__ a, const long long* __restrict__ b, size_t n, ActShape s,
                                                     size_t entries, fp2 alpha, fp2 beta, fp2 beta2, fp2 tag, const u64* __restrict__ mult,
                                                     u64* __restrict__ values, u64* __restrict__ h, int* __restrict__ err) {
    const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x, i0 = t * AB;
    if (i0 >= n) return;
    const int cnt = (int)(n - i0 < AB ? n - i0 : AB);
    fp2 d[AB], pre[AB];
    fp2 acc = f2(1, 0);
    bool zero = false;
#pragma unroll
    for (int j = 0; j < AB; j++) {
        d[j] = f2(1, 0);
        if (j < cnt) {
            const size_t i = i0 + j;
            fp2 q;
            if (mode == 0) {
                q = f2_mul_base(beta, gl_from_i64(b[i]));
                q.c0 = gl_add(q.c0, gl_add(gl_from_i64(a[i]), 2048));
                q = f2_add(q, f2_mul_base(beta2, (u64)query_group(s, i)));
            } else if (i < entries) {
                q = f2_mul_base(beta, gl_from_i64(b[i]));
                q.c0 = gl_add(q.c0, (u64)(i % 4096));
                q = f2_add(q, f2_mul_base(beta2, (u64)(i / 4096)));
            } else {
                q = f2(2048, 0);
            }
            q = f2_add(q, tag);
            if (values) *reinterpret_cast<ulonglong2*>(values + 2 * i) = make_ulonglong2(q.c0, q.c1);
            d[j] = f2_sub(alpha, q);
            zero |= f2_is_zero(d[j]);
        }
        pre[j] = acc;
        acc = f2_mul(acc, d[j]);
    }
    if (zero) { atomicExch(err, 1); return; }
    fp2 inv = f2_inv(acc);
#pragma unroll
    for (int j = AB - 1; j >= 0; j--) {
        if (j < cnt) {
            fp2 r = f2_mul(inv, pre[j]);
            if (mult) r = f2_mul_base(r, gl_canon(mult[i0 + j]));
            *reinterpret_cast<ulonglong2*>(h + 2 * (i0 + j)) = make_ulonglong2(r.c0, r.c1);
        }
        inv = f2_mul(inv, d[j]);
    }
}

struct Bufs {
    hl_ctx* c;
    std::vector<std::pair<void*, size_t>> v;
    int alloc(void** p, size_t bytes) {
        int rc = dev_alloc(c, p, bytes ? bytes : 8);
        if (!rc) v.push_back({*p, bytes ? bytes : 8});
        return rc;
    }
    ~Bufs() { for (auto& e : v) dev_free(c, e.first, e.second); }
};

bool shape_ok(size_t n, size_t f_pad, size_t tokens, size_t hidden) {
    return f_pad >= 1 && f_pad <= 0xFFFFFFFFull && tokens <= 0xFFFFFFFFull && hidden <= f_pad && n % f_pad == 0;
}

}  // namespace

extern "C" {

int hl_b200_act_histogram(hl_ctx* c, const int64_t* gates, const int64_t* outputs, size_t n, size_t f_pad, size_t tokens, size_t hidden,
                          const uint32_t* group_ids, const int64_t* tables, size_t groups, uint64_t* counts, uint64_t* misses) {
    if (!c || !gates || !outputs || !group_ids || !tables || !counts || !misses) return fail(c, HL_B200_ERR_ARG, "act_histogram: null argument");
    if (!shape_ok(n, f_pad, tokens, hidden) || groups < 1 || groups > 4) return fail(c, HL_B200_ERR_ARG, "act_histogram: query rows or table count");
    for (size_t j = 0; j < hidden; j++)
        if (group_ids[j] >= groups) return fail(c, HL_B200_ERR_ARG, "act_histogram: a group id outside the registered tables");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    Bufs bufs{c, {}};
    long long *d_g = nullptr, *d_o = nullptr, *d_t = nullptr;
    u32* d_ids = nullptr;
    unsigned long long* d_cnt = nullptr;
    const size_t nb = groups * 4096;
    int rc = bufs.alloc((void**)&d_g, n * 8);
    if (!rc) rc = bufs.alloc((void**)&d_o, n * 8);
    if (!rc) rc = bufs.alloc((void**)&d_t, nb * 8);
    if (!rc) rc = bufs.alloc((void**)&d_ids, hidden * 4);
    if (!rc) rc = bufs.alloc((void**)&d_cnt, (nb + 1) * 8);
    if (!rc) rc = h2d(c, d_g, gates, n * 8);
    if (!rc) rc = h2d(c, d_o, outputs, n * 8);
    if (!rc) rc = h2d(c, d_t, tables, nb * 8);
    if (!rc && hidden) rc = h2d(c, d_ids, group_ids, hidden * 4);
    if (!rc && cudaMemsetAsync(d_cnt, 0, (nb + 1) * 8, c->stream) != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "act_histogram: clear");
    if (!rc && n) {
        Timed t(c, HL_T_LOGUP);
        k_act_hist<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(d_g, d_o, n, ActShape{(u32)f_pad, (u32)tokens, (u32)hidden, d_ids}, d_t, (u32)groups,
                                                                      d_cnt, d_cnt + nb);
        c->stats.kernel_launches++;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "act_histogram launch", e);
    }
    if (!rc) rc = d2h(c, counts, d_cnt, nb * 8);
    if (!rc) rc = d2h(c, misses, d_cnt + nb, 8);
    if (!rc) rc = sync(c, "act_histogram");
    else cudaStreamSynchronize(c->stream);
    return rc;
}

int hl_b200_act_helpers(hl_ctx* c, const int64_t* gates, const int64_t* outputs, size_t n, size_t f_pad, size_t tokens, size_t hidden,
                        const uint32_t* group_ids, const uint64_t alpha[2], const uint64_t beta[2], const uint64_t tag[2], uint64_t* h) {
    if (!c || !gates || !outputs || !group_ids || !alpha || !beta || !tag || !h) return fail(c, HL_B200_ERR_ARG, "act_helpers: null argument");
    if (!shape_ok(n, f_pad, tokens, hidden)) return fail(c, HL_B200_ERR_ARG, "act_helpers: query rows");
    if (n == 0) return HL_B200_OK;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    Bufs bufs{c, {}};
    long long *d_g = nullptr, *d_o = nullptr;
    u32* d_ids = nullptr;
    u64* d_h = nullptr;
    int* d_err = nullptr;
    int rc = bufs.alloc((void**)&d_g, n * 8);
    if (!rc) rc = bufs.alloc((void**)&d_o, n * 8);
    if (!rc) rc = bufs.alloc((void**)&d_ids, hidden * 4);
    if (!rc) rc = bufs.alloc((void**)&d_h, n * 16);
    if (!rc) rc = bufs.alloc((void**)&d_err, 4);
    if (!rc) rc = h2d(c, d_g, gates, n * 8);
    if (!rc) rc = h2d(c, d_o, outputs, n * 8);
    if (!rc && hidden) rc = h2d(c, d_ids, group_ids, hidden * 4);
    if (!rc && cudaMemsetAsync(d_err, 0, 4, c->stream) != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "act_helpers: flag");
    const fp2 be = f2(beta[0], beta[1]);
    if (!rc) {
        Timed t(c, HL_T_LOGUP);
        const size_t threads = (n + AB - 1) / AB;
        k_act_helpers<<<(unsigned)((threads + 127) / 128), 128, 0, c->stream>>>(0, d_g, d_o, n, ActShape{(u32)f_pad, (u32)tokens, (u32)hidden, d_ids}, 0,
                                                                               f2(alpha[0], alpha[1]), be, f2_mul(be, be), f2(tag[0], tag[1]), nullptr, nullptr,
                                                                               d_h, d_err);
        c->stats.kernel_launches++;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "act_helpers launch", e);
    }
    int flag = 0;
    if (!rc) rc = d2h(c, &flag, d_err, 4);
    if (!rc) rc = sync(c, "act_helpers");
    else cudaStreamSynchronize(c->stream);
    if (!rc && flag) return fail(c, HL_B200_ERR_ZERO, "zero LogUp denominator; discard attempt");
    if (!rc) rc = d2h(c, h, d_h, n * 16);
    if (!rc) rc = sync(c, "act_helpers");
    return rc;
}

int hl_b200_act_table(hl_ctx* c, const int64_t* tables, size_t groups, size_t len, const uint64_t* mult, const uint64_t alpha[2],
                      const uint64_t beta[2], const uint64_t tag[2], uint64_t* compressed, uint64_t* ht) {
    if (!c || !tables || !mult || !alpha || !beta || !tag || !ht) return fail(c, HL_B200_ERR_ARG, "act_table: null argument");
    const size_t entries = groups * 4096;
    // table(): one to four registered tables must fit in exactly one row (accuracy_act.rs:14-17)
    if (groups < 1 || groups > 4 || len < entries || (len & (len - 1)) != 0) return fail(c, HL_B200_ERR_ARG, "act_table: one to four registered tables must fit in one row");
    for (size_t g = 0; g < groups; g++)
        if (tables[g * 4096 + 2048] != 0) return fail(c, HL_B200_ERR_ARG, "act_table: invalid generated table zero row");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    Bufs bufs{c, {}};
    long long* d_t = nullptr;
    u64 *d_m = nullptr, *d_v = nullptr, *d_h = nullptr;
    int* d_err = nullptr;
    int rc = bufs.alloc((void**)&d_t, entries * 8);
    if (!rc) rc = bufs.alloc((void**)&d_m, len * 8);
    if (!rc) rc = bufs.alloc((void**)&d_v, len * 16);
    if (!rc) rc = bufs.alloc((void**)&d_h, len * 16);
    if (!rc) rc = bufs.alloc((void**)&d_err, 4);
    if (!rc) rc = h2d(c, d_t, tables, entries * 8);
    if (!rc) rc = h2d(c, d_m, mult, len * 8);
    if (!rc && cudaMemsetAsync(d_err, 0, 4, c->stream) != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "act_table: flag");
    const fp2 be = f2(beta[0], beta[1]);
    if (!rc) {
        Timed t(c, HL_T_LOGUP);
        const size_t threads = (len + AB - 1) / AB;
        k_act_helpers<<<(unsigned)((threads + 127) / 128), 128, 0, c->stream>>>(1, nullptr, d_t, len, ActShape{1u, 0u, 0u, nullptr}, entries, f2(alpha[0], alpha[1]),
                                                                               be, f2_mul(be, be), f2(tag[0], tag[1]), d_m, d_v, d_h, d_err);
        c->stats.kernel_launches++;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "act_table launch", e);
    }
    int flag = 0;
    if (!rc) rc = d2h(c, &flag, d_err, 4);
    if (!rc) rc = sync(c, "act_table");
    else cudaStreamSynchronize(c->stream);
    if (!rc && flag) return fail(c, HL_B200_ERR_ZERO, "zero LogUp denominator; discard attempt");
    if (!rc && compressed) rc = d2h(c, compressed, d_v, len * 16);
    if (!rc) rc = d2h(c, ht, d_h, len * 16);
    if (!rc) rc = sync(c, "act_table");
    return rc;
}

}  // extern "C"
