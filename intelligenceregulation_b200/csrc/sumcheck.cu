// Sumcheck kernels: round polynomial, Fiat-Shamir step, table fold (sumcheck/rounds.rs:94-160).
//
// Tables are k arrays of `stride` Fp2 (16 bytes each); the live part of a table is its first
// `len` entries.  Variable 0 is the most significant index bit, so round j pairs entry i with
// entry i + len/2, and the fold writes the first half in place.
//
// k_sc_round   one grid pass over the pairs: each thread evaluates the slot polynomial at the
//              points 0..D by repeated addition of (T(i+half) - T(i)) and keeps D+1 running sums;
//              warp-shuffle tree, then a shared-memory tree across warps, one partial per CTA.
// k_sc_step    one warp: sums the CTA partials, recovers s(1) from the running claim, adds the
//              CFS mask c*g_j, absorbs "sc-round" into the transcript state, squeezes the
//              challenge, updates the claim and the mask's running terms (transcript.rs:67-148,
//              sumcheck.rs:260-299).  The host replays these rounds through its own transcript.
// k_sc_fold    T[i] += r (T[i+half] - T[i]) for every table, r read from device memory.
#include "b3.cuh"
#include "gl_field.cuh"
#include "kernels.h"
#include "sumcheck.h"

namespace hlk {
bool g_sc_dependent_launch = true;
void sc_set_dependent_launch(bool on) { g_sc_dependent_launch = on; }
}  // namespace hlk

namespace {

// Programmatic dependent launch: every kernel of a sumcheck is a link of one dependency chain in one stream.  A kernel opens with
// `chain_enter()`: it lets the next link be scheduled at once (its CTAs take the SM slots this grid leaves free and stop at their own
// wait) and then waits until the previous link has completed and its writes are visible.  Launched without the attribute the two
// instructions do nothing.  What the chain saves is the launch latency between dependent kernels, a few microseconds per link.
__device__ __forceinline__ void chain_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <class... P, class... A>
cudaError_t chain_launch(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, A... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = hlk::g_sc_dependent_launch ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, P(args)...);
}


using hlk::ScStep;

__device__ __forceinline__ fp2 ld2(const u64* p) {
    ulonglong2 v = *reinterpret_cast<const ulonglong2*>(p);
    return f2(v.x, v.y);
}
__device__ __forceinline__ void st2(u64* p, fp2 v) { *reinterpret_cast<ulonglong2*>(p) = make_ulonglong2(v.c0, v.c1); }

__device__ __forceinline__ fp2 f2_one() { return f2(1, 0); }

// The slot polynomial families (ids in sumcheck.h).
template <int POLY, int K>
__device__ __forceinline__ fp2 poly_eval(const fp2 (&v)[K], const fp2* __restrict__ coefs) {
    if constexpr (POLY == hlk::POLY_PROD) {
        fp2 a = v[0];
#pragma unroll
        for (int t = 1; t < K; t++) a = f2_mul(a, v[t]);
        return a;
    } else if constexpr (POLY == hlk::POLY_ZC) {
        return f2_mul(v[0], f2_sub(f2_mul(v[1], v[2]), v[3]));
    } else if constexpr (POLY == hlk::POLY_LOGUP_Q) {
        return f2_mul(v[0], f2_sub(f2_mul(v[1], f2_sub(coefs[0], v[2])), f2_one()));
    } else {
        return f2_mul(v[0], f2_sub(f2_mul(v[1], f2_sub(coefs[0], v[2])), v[3]));
    }
}

__device__ __forceinline__ u64 shfl_down64(u64 v, int d) {
    u32 lo = __shfl_down_sync(0xffffffffu, (u32)v, d), hi = __shfl_down_sync(0xffffffffu, (u32)(v >> 32), d);
    return ((u64)hi << 32) | lo;
}

constexpr int RT = 256;  // threads of a round CTA

template <int POLY, int K, int D>
__global__ void __launch_bounds__(RT) k_sc_round(const u64* __restrict__ tables, size_t stride, u32 half, const u64* __restrict__ coefs,
                                                 int eval_one, u64* __restrict__ partials) {
    chain_enter();
    fp2 acc[D + 1];
#pragma unroll
    for (int d = 0; d <= D; d++) acc[d] = f2(0, 0);
    const fp2* cf = reinterpret_cast<const fp2*>(coefs);
    for (u32 i = blockIdx.x * RT + threadIdx.x; i < half; i += gridDim.x * RT) {
        fp2 cur[K], dif[K];
#pragma unroll
        for (int t = 0; t < K; t++) {
            const u64* tb = tables + 2 * (size_t)t * stride;
            cur[t] = ld2(tb + 2 * (size_t)i);
            dif[t] = f2_sub(ld2(tb + 2 * ((size_t)i + half)), cur[t]);
        }
        acc[0] = f2_add(acc[0], poly_eval<POLY, K>(cur, cf));
#pragma unroll
        for (int d = 1; d <= D; d++) {
#pragma unroll
            for (int t = 0; t < K; t++) cur[t] = f2_add(cur[t], dif[t]);
            if (d != 1 || eval_one) acc[d] = f2_add(acc[d], poly_eval<POLY, K>(cur, cf));
        }
    }
    // warp tree
#pragma unroll
    for (int d = 0; d <= D; d++) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            acc[d].c0 = gl_add(acc[d].c0, shfl_down64(acc[d].c0, off));
            acc[d].c1 = gl_add(acc[d].c1, shfl_down64(acc[d].c1, off));
        }
    }
    __shared__ u64 wsum[RT / 32][2 * (D + 1)];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
#pragma unroll
        for (int d = 0; d <= D; d++) { wsum[warp][2 * d] = acc[d].c0; wsum[warp][2 * d + 1] = acc[d].c1; }
    }
    __syncthreads();
    if (threadIdx.x < 2 * (D + 1)) {
        u64 s = 0;
#pragma unroll
        for (int w = 0; w < RT / 32; w++) s = gl_add(s, wsum[w][threadIdx.x]);
        partials[(size_t)blockIdx.x * 2 * (D + 1) + threadIdx.x] = s;
    }
}

// ---- transcript pieces on the device: one chunk, at most 1024 bytes ----
__device__ void hash_small(const uint32_t* key, const uint32_t* words, u32 len, uint32_t (&out)[8]) {
    b3::init_cv(out, key);
    const u32 nb = len ? (len + 63) / 64 : 1;
#pragma unroll 1
    for (u32 b = 0; b < nb; b++) {
        uint32_t m[16];
#pragma unroll
        for (int i = 0; i < 16; i++) m[i] = words[16 * b + i];
        uint32_t flags = (key ? b3::KEYED : 0u) | (b == 0 ? b3::CHUNK_START : 0u) | (b == nb - 1 ? (b3::CHUNK_END | b3::ROOT) : 0u);
        b3::compress(out, m, 0, b == nb - 1 ? len - 64 * b : 64, flags);
    }
}

__device__ __forceinline__ u64 reduce_le16(const uint32_t* w) {  // 128-bit little-endian draw mod p (transcript.rs:133-148)
    return gl_reduce128(((u64)w[1] << 32) | w[0], ((u64)w[3] << 32) | w[2]);
}


// One warp.  The field work is spread over the lanes (one evaluation point per lane); only the two transcript
// hashes run on lane 0.
struct StepSmem {
    u64 sums[2 * hlk::SC_MAX_POINTS];
    u64 mskd[2 * hlk::SC_MAX_POINTS];
    u64 chal[2];
    __align__(16) uint32_t msg[64];  // 256 bytes
};

// v 2^k mod p, 0 <= k <= 62
__device__ __forceinline__ u64 gl_mul_pow2(u64 v, int k) { return gl_reduce128(v << k, k ? v >> (64 - k) : 0ull); }

__device__ __forceinline__ fp2 shfl_down8_f2(fp2 v, int d) {  // within groups of eight lanes
    u32 a0 = __shfl_down_sync(0xffffffffu, (u32)v.c0, d, 8), a1 = __shfl_down_sync(0xffffffffu, (u32)(v.c0 >> 32), d, 8);
    u32 b0 = __shfl_down_sync(0xffffffffu, (u32)v.c1, d, 8), b1 = __shfl_down_sync(0xffffffffu, (u32)(v.c1 >> 32), d, 8);
    return f2(((u64)a1 << 32) | a0, ((u64)b1 << 32) | b0);
}

// One warp; sm.sums already holds the round's D+1 sums.  The step is a serial chain (sums -> masked message -> two hashes ->
// challenge -> next claim and the mask's running terms), so it is written for depth, not for work:
//   before the hashes  one multiplication level: the mask's round polynomial is a host-made table entry plus 2^k acc_prev plus
//                      x a' prod r_i, and s_i / den_i is taken here, off the path that follows the challenge;
//   after the hashes   every lane runs the SAME product tree over eight (or four) factors and one multiplier: lanes 0..7 a
//                      Lagrange numerator prod_{j != i} (r - j) times s_i / den_i, lanes 8..15 a power r^e times the mask
//                      coefficient a_{j,e}, lane 16 the product r (a' prod r_i); sums over groups of eight lanes give the next
//                      claim (rounds.rs:145-147, mle.rs:338-351) and u_j(r_j).
// What one step reads, resolved to this round's rows and handed over by value: the step's operands then sit in registers,
// where a reference to the launch arguments would make every field a load from the local copy of the argument block.
struct StepArgs {
    int degree, round, use_claim, recover, fs, mask_vars, eval_degree;
    const fp2* aj;      // this round's `degree` mask coefficients a_{j,e}; NULL: no mask
    const fp2* tab;     // this round's degree + 1 entries of ScStep::mask_tab
    const u64* inv_den;
    const u64* extrap;  // or NULL
    hlk::ScState* state;
    u64* out;
};
__device__ __forceinline__ StepArgs step_args(const ScStep& a, int round, int use_claim, int fs, const u64* mask, const u64* mask_tab, const u64* inv_den,
                                              const u64* extrap, hlk::ScState* state) {
    StepArgs x;
    x.degree = a.degree; x.round = round; x.use_claim = use_claim; x.recover = a.recover; x.fs = fs; x.mask_vars = a.mask_vars; x.eval_degree = a.eval_degree;
    x.aj = mask ? reinterpret_cast<const fp2*>(mask) + 2 + (size_t)round * a.degree : nullptr;
    x.tab = mask ? reinterpret_cast<const fp2*>(mask_tab) + (size_t)round * (a.degree + 1) : nullptr;
    x.inv_den = inv_den; x.extrap = extrap; x.state = state; x.out = a.out;
    return x;
}

__device__ __forceinline__ void step_body(const StepArgs a, StepSmem& sm, int lane) {
    u64* sums = sm.sums;
    u64* mskd = sm.mskd;
    u64* chal = sm.chal;
    uint32_t* msg = sm.msg;
    const int np = a.degree + 1, W = 2 * np, j = a.round;
    hlk::ScState* st = a.state;
    fp2* s = reinterpret_cast<fp2*>(sums);
    if (lane == 0 && a.use_claim) s[1] = f2_sub(st->claim, s[0]);  // s(1) = claim - s(0) (rounds.rs:137-140)
    __syncwarp();
    if (a.extrap && a.eval_degree < a.degree) {
        // a polynomial of degree eval_degree is fixed by its values at 0..eval_degree: the points above, exactly
        fp2 v = f2(0, 0);
        if (lane > a.eval_degree && lane < np) {
            const u64* wrow = a.extrap + (size_t)(lane - a.eval_degree - 1) * (a.eval_degree + 1);
            for (int i = 0; i <= a.eval_degree; i++) v = f2_add(v, f2_mul_base(s[i], wrow[i]));
        }
        __syncwarp();
        if (lane > a.eval_degree && lane < np) s[lane] = v;
        __syncwarp();
    }
    u64* orow = a.out + (size_t)j * (2 * (size_t)np + 1) * 2;
    if (lane < np) st2(orow + 2 * lane, s[lane]);
    if (!a.fs) return;  // plain round(): the host drives the transcript
    const bool masked = a.aj != nullptr;
    const fp2* aj = a.aj;
    // masked message s + c g_j, one point x per lane (sumcheck.rs:260-295):
    //   g_j(x) = 2^(N-1-j) (a0 + sum_{i<j} u_i(r_i) + sum_{i>j} u_i(1)/2 + u_j(x)) + a' (prod_{i<j} r_i) x
    fp2 sd = f2(0, 0);
    if (lane < np) {
        fp2 m = s[lane];
        if (masked) {
            const fp2* tab = a.tab;
            const int sh = a.mask_vars - 1 - j;  // mask_vars <= 63
            fp2 g = f2_add(tab[lane], f2(gl_mul_pow2(st->acc_prev.c0, sh), gl_mul_pow2(st->acc_prev.c1, sh)));
            g = f2_add(g, f2_mul_base(st->ap, (u64)lane));
            m = f2_add(m, f2_mul(st->mask_c, g));
        }
        st2(mskd + 2 * lane, m);
        st2(orow + 2 * (np + lane), m);
        if (a.recover) sd = f2_mul_base(s[lane], a.inv_den[lane]);
    }
    __syncwarp();
    if (lane == 0) {
        // absorb: state' = H(state || LE64(8) || "sc-round" || LE64(16 np) || bytes) (transcript.rs:67-74)
        const uint32_t* key = st->keyed ? st->key : nullptr;
        const int nw = 14 + 2 * W;  // message words
        for (int i = nw; i < ((nw + 15) & ~15); i++) msg[i] = 0;
        for (int i = 0; i < 8; i++) msg[i] = st->state[i];
        msg[8] = 8; msg[9] = 0;
        msg[10] = 0x722d6373u; msg[11] = 0x646e756fu;  // "sc-r" "ound", little-endian words
        msg[12] = 16u * np; msg[13] = 0;
        for (int d = 0; d < W; d++) { msg[14 + 2 * d] = (uint32_t)mskd[d]; msg[15 + 2 * d] = (uint32_t)(mskd[d] >> 32); }
        uint32_t h[8];
        hash_small(key, msg, 56 + 16 * np, h);
        // squeeze: out = H(state || "squeeze" || LE64(counter)); counter++; state = out (transcript.rs:120-130)
        for (int i = 12; i < 16; i++) msg[i] = 0;
        for (int i = 0; i < 8; i++) msg[i] = h[i];
        const u64 ctr = st->counter;
        msg[8] = 0x65757173u;                                   // "sque"
        msg[9] = 0x00657a65u | ((uint32_t)(ctr & 0xff) << 24);  // "eze" then counter byte 0
        msg[10] = (uint32_t)(ctr >> 8);
        msg[11] = (uint32_t)(ctr >> 40);                        // counter bytes 5..7; the message ends there
        hash_small(key, msg, 47, h);
        st->counter = ctr + 1;
        for (int i = 0; i < 8; i++) st->state[i] = h[i];
        const fp2 r = f2(reduce_le16(h), reduce_le16(h + 4));
        chal[0] = r.c0; chal[1] = r.c1;
        st2(orow + 4 * np, r);
        st->r = r;
    }
    __syncwarp();
    if (!a.recover && !masked) return;
    const fp2 r = f2(chal[0], chal[1]);
    const int grp = lane >> 3, li = lane & 7;
    fp2 f[8], mult = f2(0, 0);
#pragma unroll
    for (int t = 0; t < 8; t++) f[t] = f2_one();
    if (grp == 0) {
        if (a.recover && li < np) {
#pragma unroll
            for (int t = 0; t < 7; t++) {  // the points other than li, in order
                const int jj = t < li ? t : t + 1;
                if (jj < np) f[t] = f2(gl_sub(r.c0, (u64)jj), r.c1);
            }
            mult = sd;
        }
    } else if (grp == 1) {
        if (masked && li < a.degree) {  // r^(li + 1) a_{j, li + 1}
#pragma unroll
            for (int t = 0; t < 7; t++)
                if (t <= li) f[t] = r;
            mult = aj[li];
        }
    } else if (lane == 16 && masked) {
        f[0] = r;
        f[1] = st->ap;
        mult = f2_one();
    }
    fp2 prod = f2_mul(f2_mul(f[0], f[1]), f2_mul(f[2], f[3]));
    if (a.degree > 4) prod = f2_mul(prod, f2_mul(f2_mul(f[4], f[5]), f2_mul(f[6], f[7])));
    fp2 term = f2_mul(prod, mult);
    const fp2 own = term;
#pragma unroll
    for (int off = 4; off >= 1; off >>= 1) term = f2_add(term, shfl_down8_f2(term, off));
    if (lane == 0 && a.recover) st->claim = term;
    if (lane == 8 && masked) st->acc_prev = f2_add(st->acc_prev, term);
    if (lane == 16 && masked) st->ap = own;
}

// The CTA partials of a round are summed by all STEP_T threads (independent loads, shared-memory tree);
// warp 0 then runs the Fiat-Shamir step.
constexpr int STEP_T = 512;
__global__ void __launch_bounds__(STEP_T) k_sc_step(ScStep a) {
    chain_enter();
    __shared__ StepSmem sm;
    __shared__ u64 red[STEP_T];
    // everything the serial step reads is fetched by the whole CTA while the partials are summed: the step itself then waits on
    // no global load (each one is most of a microsecond for a single warp)
    __shared__ hlk::ScState st_s;
    __shared__ u64 row_s[2 * hlk::SC_MAX_POINTS], tab_s[2 * hlk::SC_MAX_POINTS], invden_s[hlk::SC_MAX_POINTS], extrap_s[hlk::SC_MAX_POINTS * hlk::SC_MAX_POINTS];
    hlk::ScState* const st_global = a.state;
    {
        const u32* src = reinterpret_cast<const u32*>(a.state);
        u32* dst = reinterpret_cast<u32*>(&st_s);
        if (threadIdx.x < sizeof(hlk::ScState) / 4) dst[threadIdx.x] = src[threadIdx.x];
        const int t = (int)threadIdx.x - 64;
        if (a.mask && a.fs) {
            if (t >= 0 && t < 2 * a.degree) row_s[t] = a.mask[4 + 2 * (size_t)a.round * a.degree + t];
            if (t >= 16 && t < 16 + 2 * (a.degree + 1)) tab_s[t - 16] = a.mask_tab[2 * (size_t)a.round * (a.degree + 1) + (t - 16)];
        }
        if (t >= 40 && t < 40 + a.degree + 1) invden_s[t - 40] = a.inv_den[t - 40];
        const int ne = a.extrap ? (a.degree - a.eval_degree) * (a.eval_degree + 1) : 0;
        if (t >= 64 && t < 64 + ne) extrap_s[t - 64] = a.extrap[t - 64];
    }
    const int W = 2 * (a.degree + 1);              // <= 16 words per partial row
    const int w = threadIdx.x & 15, grp = threadIdx.x >> 4;  // STEP_T / 16 groups stride over the rows
    u64 s = 0;
    if (w < W) {
#pragma unroll 4
        for (u32 b = grp; b < a.nblocks; b += STEP_T / 16) s = gl_add(s, a.partials[(size_t)b * W + w]);
    }
    red[threadIdx.x] = s;
    __syncthreads();
    for (int stride = STEP_T / 2; stride >= 16; stride >>= 1) {
        if (threadIdx.x < stride) red[threadIdx.x] = gl_add(red[threadIdx.x], red[threadIdx.x + stride]);
        __syncthreads();
    }
    if (threadIdx.x < W) sm.sums[threadIdx.x] = red[threadIdx.x];
    __syncthreads();
    if (threadIdx.x < 32) {
        StepArgs x = step_args(a, a.round, a.use_claim, a.fs, nullptr, nullptr, invden_s, a.extrap ? extrap_s : nullptr, &st_s);
        if (a.mask && a.fs) { x.aj = reinterpret_cast<const fp2*>(row_s); x.tab = reinterpret_cast<const fp2*>(tab_s); }
        step_body(x, sm, threadIdx.x);
        __syncwarp();
        const u32* src = reinterpret_cast<const u32*>(&st_s);
        u32* dst = reinterpret_cast<u32*>(st_global);
        for (u32 i = threadIdx.x; i < sizeof(hlk::ScState) / 4; i += 32) dst[i] = src[i];
    }
}

// The tail of a sumcheck in ONE CTA: once a round has at most TAIL_HALF pairs, the remaining rounds (round sums,
// Fiat-Shamir step, fold) run back to back behind block barriers instead of three launches per round.
constexpr int TAIL_T = 1024;
template <int POLY, int K, int D>
__global__ void __launch_bounds__(TAIL_T) k_sc_tail(u64* __restrict__ tables, size_t stride, u32 len, const u64* __restrict__ coefs,
                                                    ScStep a, int nrounds, int first_has_claim, u64* __restrict__ scratch) {
    chain_enter();
    __shared__ StepSmem sm;
    __shared__ u64 wsum[TAIL_T / 32][2 * (D + 1)];
    // the evaluator state, the mask and the Lagrange denominators stay in shared memory for the whole tail:
    // the serial step then waits on no global load
    __shared__ hlk::ScState st_s;
    __shared__ u64 mask_s[2 * (63 * D + 2)];
    __shared__ u64 tab_s[2 * 63 * (D + 1)];
    __shared__ u64 invden_s[hlk::SC_MAX_POINTS];
    const fp2* cf = reinterpret_cast<const fp2*>(coefs);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    {
        const u32* src = reinterpret_cast<const u32*>(a.state);
        u32* dst = reinterpret_cast<u32*>(&st_s);
        for (u32 i = threadIdx.x; i < sizeof(hlk::ScState) / 4; i += TAIL_T) dst[i] = src[i];
        if (a.mask) {
            for (u32 i = threadIdx.x; i < 2u * (a.mask_vars * D + 2); i += TAIL_T) mask_s[i] = a.mask[i];
            for (u32 i = threadIdx.x; i < 2u * a.mask_vars * (D + 1); i += TAIL_T) tab_s[i] = a.mask_tab[i];
        }
        if (threadIdx.x <= D) invden_s[threadIdx.x] = a.inv_den[threadIdx.x];
    }
    hlk::ScState* const st_global = a.state;
    const u64* const mask_p = a.mask ? mask_s : nullptr;
    __syncthreads();
    for (int rd = 0; rd < nrounds; rd++) {
        const u32 half = len >> 1;
        const bool have_claim = a.recover && (rd > 0 || first_has_claim);
        // warps beyond the round's pairs hold nothing: they skip the sums and their reduction (32 warps reducing zeros cost more
        // than the round's arithmetic once a round is down to a few pairs)
        const u32 live_warps = (half + 31u) >> 5 < (u32)(TAIL_T / 32) ? (half + 31u) >> 5 : (u32)(TAIL_T / 32);
        if ((u32)warp < live_warps) {
            fp2 acc[D + 1];
#pragma unroll
            for (int d = 0; d <= D; d++) acc[d] = f2(0, 0);
            for (u32 i = threadIdx.x; i < half; i += TAIL_T) {
                fp2 cur[K], dif[K];
#pragma unroll
                for (int t = 0; t < K; t++) {
                    const u64* tb = tables + 2 * (size_t)t * stride;
                    cur[t] = ld2(tb + 2 * (size_t)i);
                    dif[t] = f2_sub(ld2(tb + 2 * ((size_t)i + half)), cur[t]);
                }
                acc[0] = f2_add(acc[0], poly_eval<POLY, K>(cur, cf));
#pragma unroll
                for (int d = 1; d <= D; d++) {
#pragma unroll
                    for (int t = 0; t < K; t++) cur[t] = f2_add(cur[t], dif[t]);
                    if (d != 1 || !have_claim) acc[d] = f2_add(acc[d], poly_eval<POLY, K>(cur, cf));
                }
            }
#pragma unroll
            for (int d = 0; d <= D; d++) {
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
                    acc[d].c0 = gl_add(acc[d].c0, shfl_down64(acc[d].c0, off));
                    acc[d].c1 = gl_add(acc[d].c1, shfl_down64(acc[d].c1, off));
                }
            }
            if (lane == 0) {
#pragma unroll
                for (int d = 0; d <= D; d++) { wsum[warp][2 * d] = acc[d].c0; wsum[warp][2 * d + 1] = acc[d].c1; }
            }
        }
        __syncthreads();
        if (threadIdx.x < 2 * (D + 1)) {
            u64 s = 0;
            for (u32 w = 0; w < live_warps; w++) s = gl_add(s, wsum[w][threadIdx.x]);
            sm.sums[threadIdx.x] = s;
        }
        __syncthreads();
        if (warp == 0) step_body(step_args(a, a.round + rd, have_claim ? 1 : 0, 1, mask_p, tab_s, invden_s, a.extrap, &st_s), sm, lane);
        __syncthreads();
        const fp2 r = st_s.r;
        for (u32 x = threadIdx.x; x < half * K; x += TAIL_T) {
            const u32 t = x / half, i = x - t * half;
            u64* tb = tables + 2 * (size_t)t * stride;
            fp2 p = ld2(tb + 2 * (size_t)i), q = ld2(tb + 2 * ((size_t)i + half));
            st2(tb + 2 * (size_t)i, f2_add(p, f2_mul(r, f2_sub(q, p))));
        }
        __syncthreads();
        len = half;
    }
    {
        const u32* src = reinterpret_cast<const u32*>(&st_s);
        u32* dst = reinterpret_cast<u32*>(st_global);
        for (u32 i = threadIdx.x; i < sizeof(hlk::ScState) / 4; i += TAIL_T) dst[i] = src[i];
    }
}

// which tables are extension-valued: one CTA row per table, the second words OR-ed
__global__ void __launch_bounds__(256) k_sc_nonbase(const u64* __restrict__ tables, size_t stride, size_t len, u64* __restrict__ mask) {
    const u32 t = blockIdx.y;
    const u64* tb = tables + 2 * (size_t)t * stride;
    u64 any = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += (size_t)gridDim.x * blockDim.x) any |= tb[2 * i + 1];
    if (__syncthreads_or(any != 0) && threadIdx.x == 0) atomicOr(mask, 1ull << t);
}

// The fold with the previous challenge and the sums of the next round in ONE pass (the closed-form families): the tables are
// stored at length 2 n, unfolded; a thread reads T[i], T[i + n], T[i + half], T[i + half + n] (half = n / 2), writes the two
// folded entries T[i], T[i + half] - no other thread reads or writes those four places - and evaluates the round polynomial
// on them.  A table word is read once and written once per round, and a round is two launches (this one and the step).
template <int POLY, int K, int D>
__global__ void __launch_bounds__(RT) k_sc_fold_round(u64* __restrict__ tables, size_t stride, u32 n, const u64* __restrict__ coefs,
                                                      const hlk::ScState* __restrict__ st, int eval_one, u64* __restrict__ partials) {
    chain_enter();
    fp2 acc[D + 1];
#pragma unroll
    for (int d = 0; d <= D; d++) acc[d] = f2(0, 0);
    const fp2* cf = reinterpret_cast<const fp2*>(coefs);
    const fp2 r = st->r;
    const u32 half = n >> 1;
    for (u32 i = blockIdx.x * RT + threadIdx.x; i < half; i += gridDim.x * RT) {
        fp2 cur[K], dif[K];
#pragma unroll
        for (int t = 0; t < K; t++) {
            u64* tb = tables + 2 * (size_t)t * stride;
            const fp2 a0 = ld2(tb + 2 * (size_t)i), a1 = ld2(tb + 2 * ((size_t)i + n));
            const fp2 b0 = ld2(tb + 2 * ((size_t)i + half)), b1 = ld2(tb + 2 * ((size_t)i + half + n));
            const fp2 lo = f2_add(a0, f2_mul(r, f2_sub(a1, a0))), hi = f2_add(b0, f2_mul(r, f2_sub(b1, b0)));
            st2(tb + 2 * (size_t)i, lo);
            st2(tb + 2 * ((size_t)i + half), hi);
            cur[t] = lo;
            dif[t] = f2_sub(hi, lo);
        }
        acc[0] = f2_add(acc[0], poly_eval<POLY, K>(cur, cf));
#pragma unroll
        for (int d = 1; d <= D; d++) {
#pragma unroll
            for (int t = 0; t < K; t++) cur[t] = f2_add(cur[t], dif[t]);
            if (d != 1 || eval_one) acc[d] = f2_add(acc[d], poly_eval<POLY, K>(cur, cf));
        }
    }
#pragma unroll
    for (int d = 0; d <= D; d++) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            acc[d].c0 = gl_add(acc[d].c0, shfl_down64(acc[d].c0, off));
            acc[d].c1 = gl_add(acc[d].c1, shfl_down64(acc[d].c1, off));
        }
    }
    __shared__ u64 wsum[RT / 32][2 * (D + 1)];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
#pragma unroll
        for (int d = 0; d <= D; d++) { wsum[warp][2 * d] = acc[d].c0; wsum[warp][2 * d + 1] = acc[d].c1; }
    }
    __syncthreads();
    if (threadIdx.x < 2 * (D + 1)) {
        u64 s = 0;
#pragma unroll
        for (int w = 0; w < RT / 32; w++) s = gl_add(s, wsum[w][threadIdx.x]);
        partials[(size_t)blockIdx.x * 2 * (D + 1) + threadIdx.x] = s;
    }
}

__global__ void __launch_bounds__(256) k_sc_fold(u64* __restrict__ tables, size_t stride, u32 half, u32 k, const hlk::ScState* __restrict__ st) {
    chain_enter();
    const u32 i = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (i >= half || t >= k) return;
    const fp2 r = st->r;
    u64* tb = tables + 2 * (size_t)t * stride;
    fp2 a = ld2(tb + 2 * (size_t)i), b = ld2(tb + 2 * ((size_t)i + half));
    st2(tb + 2 * (size_t)i, f2_add(a, f2_mul(r, f2_sub(b, a))));
}


// ---------------------------------------------------------------------------------------------
// Slot polynomials given as data (slot_ir.cuh): the same round / tail structure with the polynomial
// interpreted from its evaluation plan, held in shared memory.  Two forms:
//   pair form    one PAIR per warp, every evaluation point at once.  Table values and affine nodes are stepped
//                along the round's variable by additions; the remaining nodes run level by level with one
//                (unit, point) product per lane, then one (node, point) sum per lane.  All values stay in shared
//                memory (a 60-table, 70-node polynomial keeps ~19 KB per warp), nothing spills, and a pair costs
//                microseconds, so the same kernel serves the long rounds and the short ones.
//   thread form  one (pair, point) per thread with the values in local memory: polynomials of a few units, where
//                a warp would idle.
// ---------------------------------------------------------------------------------------------
constexpr int IRT = 128;             // thread form
constexpr int IRC_MAX_WARPS = 8;     // pair form, warps per CTA (fewer when the areas are large)
constexpr int IR_TAIL_T = 512;       // single-CTA tail, thread form (the pair form uses as many warps as fit)

__device__ __forceinline__ void ir_stage(const hlk::IrDev& p, u32* w_s, fp2*& cf_s, int nthreads) {
    for (u32 x = threadIdx.x; x < p.plan_words; x += nthreads) w_s[x] = p.plan[x];
    cf_s = reinterpret_cast<fp2*>(w_s + ((p.plan_words + 3u) & ~3u));
    for (u32 x = threadIdx.x; x < p.n_coefs; x += nthreads) cf_s[x] = ld2(p.coefs + 2 * (size_t)x);
}

__device__ __forceinline__ fp2 ir_table_value(const u64* __restrict__ tb, u32 i, u32 half, u32 d) {
    if (d == 0) return ld2(tb + 2 * (size_t)i);
    if (d == 1) return ld2(tb + 2 * ((size_t)i + half));
    const fp2 lo = ld2(tb + 2 * (size_t)i), hi = ld2(tb + 2 * ((size_t)i + half));
    return f2_add(lo, f2_mul_base(f2_sub(hi, lo), (u64)d));
}

// thread form: grid (blocks, degree + 1), row y evaluates point y; partials[block][point] as in k_sc_round
__global__ void __launch_bounds__(IRT) k_sc_round_ir(const u64* __restrict__ tables, size_t stride, u32 half, hlk::IrDev p, int degree,
                                                     int eval_one, u64* __restrict__ partials) {
    chain_enter();
    extern __shared__ __align__(16) u32 ir_smem[];
    __shared__ u64 wsum[IRT / 32][2];
    fp2* cf_s;
    const u32 d = blockIdx.y;
    u64* dst = partials + ((size_t)blockIdx.x * (degree + 1) + d) * 2;
    if (d == 1 && !eval_one) {  // s(1) comes from the running claim
        if (threadIdx.x < 2) dst[threadIdx.x] = 0;
        return;
    }
    ir_stage(p, ir_smem, cf_s, IRT);
    __syncthreads();
    fp2 tv[ir::MAX_TABLES], nv[ir::MAX_NODES + 1];
    fp2 acc = f2(0, 0);
    for (u32 i = blockIdx.x * IRT + threadIdx.x; i < half; i += gridDim.x * IRT) {
        for (u32 t = 0; t < p.n_tables; t++) tv[t] = ir_table_value(tables + 2 * (size_t)t * stride, i, half, d);
        acc = f2_add(acc, ir::plan_eval(ir_smem, cf_s, tv, nv));
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        acc.c0 = gl_add(acc.c0, shfl_down64(acc.c0, off));
        acc.c1 = gl_add(acc.c1, shfl_down64(acc.c1, off));
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { wsum[warp][0] = acc.c0; wsum[warp][1] = acc.c1; }
    __syncthreads();
    if (threadIdx.x < 2) {
        u64 s = 0;
#pragma unroll
        for (int w = 0; w < IRT / 32; w++) s = gl_add(s, wsum[w][threadIdx.x]);
        dst[threadIdx.x] = s;
    }
}

// thread pair form: one pair per thread, every point; only live tables and node values are kept (slot_ir.cuh).  The long
// rounds: it evaluates the affine nodes once per pair instead of once per point and needs no interpolation of the tables.
constexpr u32 IRP_VALUES = ir::MAX_TABLES + ir::MAX_NODES + 1;
__global__ void __launch_bounds__(IRT, 8) k_sc_round_irp(const u64* __restrict__ tables, size_t stride, u32 half, hlk::IrDev p, int degree,
                                                      int eval_one, u64* __restrict__ partials) {
    chain_enter();
    extern __shared__ __align__(16) u32 ir_smem[];
    __shared__ u64 wsum[IRT / 32][2 * hlk::SC_MAX_POINTS];
    fp2* cf_s;
    ir_stage(p, ir_smem, cf_s, IRT);
    __syncthreads();
    const u32* pw = ir_smem;
    const u32 nl = pw[14];
    const u32* live = pw + pw[13];
    fp2 V[IRP_VALUES], D[IRP_VALUES];
    fp2 acc[hlk::SC_MAX_POINTS];
#pragma unroll
    for (int d = 0; d < hlk::SC_MAX_POINTS; d++) acc[d] = f2(0, 0);
    for (u32 i = blockIdx.x * IRT + threadIdx.x; i < half; i += gridDim.x * IRT) {
        for (u32 j = 0; j < nl; j++) {
            const u64* tb = tables + 2 * (size_t)live[j] * stride;
            V[j] = ld2(tb + 2 * (size_t)i);
            D[j] = f2_sub(ld2(tb + 2 * ((size_t)i + half)), V[j]);
        }
        ir::tpair_affine(pw, cf_s, V, D, [&](u32 t, fp2& lo, fp2& df) {
            const u64* tb = tables + 2 * (size_t)t * stride;
            lo = ld2(tb + 2 * (size_t)i);
            df = f2_sub(ld2(tb + 2 * ((size_t)i + half)), lo);
        });
        acc[0] = f2_add(acc[0], ir::tpair_sums(pw, cf_s, V));
        for (int d = 1; d <= (int)p.eval_degree; d++) {
            ir::tpair_step(pw, V, D);
            if (d == 1 && !eval_one) continue;
            const fp2 v = ir::tpair_sums(pw, cf_s, V);
#pragma unroll
            for (int dd = 1; dd < hlk::SC_MAX_POINTS; dd++)
                if (dd == d) acc[dd] = f2_add(acc[dd], v);
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, np = degree + 1;
    for (int d = 0; d < np; d++) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            acc[d].c0 = gl_add(acc[d].c0, shfl_down64(acc[d].c0, off));
            acc[d].c1 = gl_add(acc[d].c1, shfl_down64(acc[d].c1, off));
        }
    }
    if (lane == 0) {
        for (int d = 0; d < np; d++) { wsum[warp][2 * d] = acc[d].c0; wsum[warp][2 * d + 1] = acc[d].c1; }
    }
    __syncthreads();
    if ((int)threadIdx.x < 2 * np) {
        u64 s = 0;
#pragma unroll
        for (int w = 0; w < IRT / 32; w++) s = gl_add(s, wsum[w][threadIdx.x]);
        partials[(size_t)blockIdx.x * 2 * np + threadIdx.x] = s;
    }
}

// The same with every unit evaluated at all points at once (slot_ir.cuh tpair_sums_all): a fifth of the record decoding
// and of the value loads, and independent product chains per point.  For plans within its fixed array sizes.
template <u32 NPW, bool SKIP>
__global__ void __launch_bounds__(IRT, 4) k_sc_round_irq(const u64* __restrict__ tables, size_t stride, u32 half, hlk::IrDev p, int degree,
                                                         u64* __restrict__ partials) {
    chain_enter();
    extern __shared__ __align__(16) u32 ir_smem[];
    __shared__ u64 wsum[IRT / 32][2 * hlk::SC_MAX_POINTS];
    fp2* cf_s;
    ir_stage(p, ir_smem, cf_s, IRT);
    __syncthreads();
    const u32* pw = ir_smem;
    const u32 nl = pw[14];
    const u32* live = pw + pw[13];
    fp2 V[ir::TPAIR_AFFINE_VALUES], D[ir::TPAIR_AFFINE_VALUES], W[ir::TPAIR_SUM_NODES * NPW];
    fp2 acc[ir::TPAIR_POINTS];
#pragma unroll
    for (u32 d = 0; d < ir::TPAIR_POINTS; d++) acc[d] = f2(0, 0);
    for (u32 i = blockIdx.x * IRT + threadIdx.x; i < half; i += gridDim.x * IRT) {
        for (u32 j = 0; j < nl; j++) {
            const u64* tb = tables + 2 * (size_t)live[j] * stride;
            V[j] = ld2(tb + 2 * (size_t)i);
            D[j] = f2_sub(ld2(tb + 2 * ((size_t)i + half)), V[j]);
        }
        ir::tpair_affine(pw, cf_s, V, D, [&](u32 t, fp2& lo, fp2& df) {
            const u64* tb = tables + 2 * (size_t)t * stride;
            lo = ld2(tb + 2 * (size_t)i);
            df = f2_sub(ld2(tb + 2 * ((size_t)i + half)), lo);
        });
        fp2 res[ir::TPAIR_POINTS];
        ir::tpair_sums_all_t<NPW, SKIP>(pw, cf_s, V, D, W, res);
#pragma unroll
        for (u32 d = 0; d < ir::TPAIR_POINTS; d++) acc[d] = f2_add(acc[d], res[d]);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, np = degree + 1;
#pragma unroll
    for (u32 d = 0; d < ir::TPAIR_POINTS; d++) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            acc[d].c0 = gl_add(acc[d].c0, shfl_down64(acc[d].c0, off));
            acc[d].c1 = gl_add(acc[d].c1, shfl_down64(acc[d].c1, off));
        }
    }
    if (lane < 2 * hlk::SC_MAX_POINTS) wsum[warp][lane] = 0;
    __syncwarp();
    if (lane == 0) {
#pragma unroll
        for (u32 d = 0; d < ir::TPAIR_POINTS; d++) { wsum[warp][2 * d] = acc[d].c0; wsum[warp][2 * d + 1] = acc[d].c1; }
    }
    __syncthreads();
    if ((int)threadIdx.x < 2 * np) {
        u64 s = 0;
#pragma unroll
        for (int w = 0; w < IRT / 32; w++) s = gl_add(s, wsum[w][threadIdx.x]);
        partials[(size_t)blockIdx.x * 2 * np + threadIdx.x] = s;
    }
}

// pair form, one pair by one warp; afterwards V holds the final node's value at every evaluated point
__device__ __forceinline__ void ir_pair_item(const ir::Pair& a, const u64* __restrict__ tables, size_t stride, u32 i, u32 half, u32 lane) {
    for (u32 t = lane; t < a.n_tables; t += 32) {
        const u64* tb = tables + 2 * (size_t)t * stride;
        const fp2 lo = ld2(tb + 2 * (size_t)i);
        a.V[t * a.np] = lo;
        a.DV[t] = f2_sub(ld2(tb + 2 * ((size_t)i + half)), lo);
    }
    __syncwarp();
    for (u32 g = 0; g < a.pw[11]; g++) {
        ir::pair_affine_units(a, g, lane, 32);
        __syncwarp();
        ir::pair_affine_nodes(a, g, lane, 32);
        __syncwarp();
    }
    ir::pair_step(a, lane, 32);
    __syncwarp();
    for (u32 l = 0; l < a.pw[0]; l++) {
        ir::pair_level_units(a, l, lane, 32);
        __syncwarp();
        ir::pair_level_nodes(a, l, lane, 32);
        __syncwarp();
    }
}

__device__ __forceinline__ ir::Pair ir_pair_setup(const hlk::IrDev& p, const u32* pw_s, fp2* cf_s, u32 warp, int degree, bool skip_one) {
    ir::Pair a;
    (void)degree;
    const u32 np = p.eval_degree + 1, ids = p.n_tables + p.n_nodes;
    fp2* area = cf_s + p.n_coefs + (size_t)warp * ir::pair_area(p.n_tables, p.n_nodes, np);
    a.pw = pw_s; a.cf = cf_s; a.V = area; a.DV = area + (size_t)ids * np; a.UB = a.DV + ids;
    a.n_tables = p.n_tables; a.np = np; a.npe = skip_one ? np - 1 : np;
    return a;
}

__global__ void __launch_bounds__(IRC_MAX_WARPS * 32) k_sc_round_irc(const u64* __restrict__ tables, size_t stride, u32 half, hlk::IrDev p,
                                                                     int degree, int eval_one, u64* __restrict__ partials) {
    chain_enter();
    extern __shared__ __align__(16) u32 ir_smem[];
    __shared__ u64 wsum[IRC_MAX_WARPS][2 * hlk::SC_MAX_POINTS];
    fp2* cf_s;
    ir_stage(p, ir_smem, cf_s, blockDim.x);
    __syncthreads();
    const u32 lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5, np = (u32)degree + 1;
    const ir::Pair a = ir_pair_setup(p, ir_smem, cf_s, warp, degree, !eval_one && p.eval_degree >= 1);
    const u32 fin = (p.n_tables + p.n_nodes - 1) * a.np;  // the final node's values
    fp2 acc = f2(0, 0);  // lane pi: the sum at evaluated point pi
    for (u32 i = blockIdx.x * nwarps + warp; i < half; i += gridDim.x * nwarps) {
        ir_pair_item(a, tables, stride, i, half, lane);
        if (lane < a.npe) acc = f2_add(acc, a.V[fin + a.point(lane)]);
        __syncwarp();
    }
    if (lane < 2 * hlk::SC_MAX_POINTS) wsum[warp][lane] = 0;
    __syncwarp();
    if (lane < a.npe) { wsum[warp][2 * a.point(lane)] = acc.c0; wsum[warp][2 * a.point(lane) + 1] = acc.c1; }
    __syncthreads();
    if (threadIdx.x < 2 * np) {
        u64 s = 0;
        for (u32 w = 0; w < nwarps; w++) s = gl_add(s, wsum[w][threadIdx.x]);
        partials[(size_t)blockIdx.x * 2 * np + threadIdx.x] = s;
    }
}

template <bool PAIR_FORM>
__global__ void __launch_bounds__(IR_TAIL_T) k_sc_tail_ir(u64* __restrict__ tables, size_t stride, u32 len, hlk::IrDev p, int degree, int k,
                                                          ScStep a, int nrounds, int first_has_claim) {
    chain_enter();
    extern __shared__ __align__(16) u32 ir_smem[];
    __shared__ StepSmem sm;
    __shared__ u64 wsum[IR_TAIL_T / 32][2 * hlk::SC_MAX_POINTS];
    __shared__ hlk::ScState st_s;
    __shared__ u64 mask_s[2 * (63 * (hlk::SC_MAX_POINTS - 1) + 2)];
    __shared__ u64 tab_s[2 * 63 * hlk::SC_MAX_POINTS];
    __shared__ u64 invden_s[hlk::SC_MAX_POINTS];
    __shared__ u64 extrap_s[hlk::SC_MAX_POINTS * hlk::SC_MAX_POINTS];
    fp2* cf_s;
    const u32 nthreads = blockDim.x, nwarps = nthreads >> 5;
    ir_stage(p, ir_smem, cf_s, nthreads);
    const u32 lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int np = degree + 1;
    {
        const u32* src = reinterpret_cast<const u32*>(a.state);
        u32* dst = reinterpret_cast<u32*>(&st_s);
        for (u32 i = threadIdx.x; i < sizeof(hlk::ScState) / 4; i += nthreads) dst[i] = src[i];
        if (a.mask) {
            for (u32 i = threadIdx.x; i < 2u * (a.mask_vars * degree + 2); i += nthreads) mask_s[i] = a.mask[i];
            for (u32 i = threadIdx.x; i < 2u * a.mask_vars * np; i += nthreads) tab_s[i] = a.mask_tab[i];
        }
        if ((int)threadIdx.x < np) invden_s[threadIdx.x] = a.inv_den[threadIdx.x];
        if (a.extrap && (int)threadIdx.x < (a.degree - a.eval_degree) * (a.eval_degree + 1)) extrap_s[threadIdx.x] = a.extrap[threadIdx.x];
    }
    hlk::ScState* const st_global = a.state;
    const u64* const mask_p = a.mask ? mask_s : nullptr;
    const u64* const extrap_p = a.extrap ? extrap_s : nullptr;
    __syncthreads();
    for (int rd = 0; rd < nrounds; rd++) {
        const u32 half = len >> 1;  // a power of two
        const bool have_claim = a.recover && (rd > 0 || first_has_claim);
        if (threadIdx.x < 2 * hlk::SC_MAX_POINTS)
            for (u32 w = 0; w < nwarps; w++) wsum[w][threadIdx.x] = 0;
        __syncthreads();
        if constexpr (PAIR_FORM) {
            const ir::Pair pa = ir_pair_setup(p, ir_smem, cf_s, warp, degree, have_claim && p.eval_degree >= 1);
            const u32 fin = (p.n_tables + p.n_nodes - 1) * pa.np;
            fp2 acc = f2(0, 0);
            for (u32 i = warp; i < half; i += nwarps) {
                ir_pair_item(pa, tables, stride, i, half, lane);
                if (lane < pa.npe) acc = f2_add(acc, pa.V[fin + pa.point(lane)]);
                __syncwarp();
            }
            if (lane < pa.npe) { wsum[warp][2 * pa.point(lane)] = acc.c0; wsum[warp][2 * pa.point(lane) + 1] = acc.c1; }
        } else {
            fp2 acc[hlk::SC_MAX_POINTS];
#pragma unroll
            for (int d = 0; d < hlk::SC_MAX_POINTS; d++) acc[d] = f2(0, 0);
            fp2 tv[ir::MAX_TABLES], nv[ir::MAX_NODES + 1];
            for (u32 x = threadIdx.x; x < half * (p.eval_degree + 1); x += nthreads) {
                const u32 d = x / half, i = x - d * half;
                if (d == 1 && have_claim) continue;
                for (u32 t = 0; t < p.n_tables; t++) tv[t] = ir_table_value(tables + 2 * (size_t)t * stride, i, half, d);
                const fp2 v = ir::plan_eval(ir_smem, cf_s, tv, nv);
#pragma unroll
                for (int dd = 0; dd < hlk::SC_MAX_POINTS; dd++)
                    if ((u32)dd == d) acc[dd] = f2_add(acc[dd], v);
            }
            for (int d = 0; d < np; d++) {
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
                    acc[d].c0 = gl_add(acc[d].c0, shfl_down64(acc[d].c0, off));
                    acc[d].c1 = gl_add(acc[d].c1, shfl_down64(acc[d].c1, off));
                }
            }
            if (lane == 0) {
                for (int d = 0; d < np; d++) { wsum[warp][2 * d] = acc[d].c0; wsum[warp][2 * d + 1] = acc[d].c1; }
            }
        }
        __syncthreads();
        if ((int)threadIdx.x < 2 * np) {
            u64 s = 0;
            for (u32 w = 0; w < nwarps; w++) s = gl_add(s, wsum[w][threadIdx.x]);
            sm.sums[threadIdx.x] = s;
        }
        __syncthreads();
        if (warp == 0) step_body(step_args(a, a.round + rd, have_claim ? 1 : 0, 1, mask_p, tab_s, invden_s, extrap_p, &st_s), sm, (int)lane);
        __syncthreads();
        const fp2 r = st_s.r;
        for (u32 x = threadIdx.x; x < half * (u32)k; x += nthreads) {
            const u32 t = x / half, i = x - t * half;
            u64* tb = tables + 2 * (size_t)t * stride;
            fp2 lo = ld2(tb + 2 * (size_t)i), hi = ld2(tb + 2 * ((size_t)i + half));
            st2(tb + 2 * (size_t)i, f2_add(lo, f2_mul(r, f2_sub(hi, lo))));
        }
        __syncthreads();
        len = half;
    }
    {
        const u32* src = reinterpret_cast<const u32*>(&st_s);
        u32* dst = reinterpret_cast<u32*>(st_global);
        for (u32 i = threadIdx.x; i < sizeof(hlk::ScState) / 4; i += nthreads) dst[i] = src[i];
    }
}

// A polynomial of few units leaves most lanes of a warp idle: it stays in the thread form.  So do the long rounds of
// every polynomial: with more (pair, point) items than resident threads the thread form is bound by instruction
// throughput, where it needs a third of the pair form's warp instructions (no idle lanes); measured on the 219-unit
// graph it takes 2.5 ns per item (12.5 ns per pair) from 2^15 pairs up, the pair form 28 ns per pair but only
// ~43 us for a whole short round, where one thread needs 120-290 us for its single item.
bool ir_pair_capable(const hlk::IrDev& p) { return p.n_units >= 24; }
bool ir_pair_form(const hlk::IrDev& p, u32 half) { return ir_pair_capable(p) && half < (1u << 14); }
// the long rounds of a large polynomial: one pair per thread
bool ir_thread_pair_form(const hlk::IrDev& p, u32 half) { return ir_pair_capable(p) && half >= (1u << 14); }
constexpr size_t IR_SMEM_BUDGET = 200 * 1024;
size_t ir_fixed_bytes(const hlk::IrDev& p) { return (((size_t)p.plan_words + 3) & ~(size_t)3) * 4 + (size_t)p.n_coefs * 16 + 16; }
size_t ir_area_bytes(const hlk::IrDev& p, int degree) { (void)degree; return (size_t)ir::pair_area(p.n_tables, p.n_nodes, p.eval_degree + 1) * 16; }
// warps of a pair-form CTA: as many as the shared memory holds, at most `want`
int ir_pair_warps(const hlk::IrDev& p, int degree, int want) {
    const size_t fixed = ir_fixed_bytes(p), area = ir_area_bytes(p, degree);
    if (fixed + area > IR_SMEM_BUDGET) return 0;
    const size_t fit = (IR_SMEM_BUDGET - fixed) / area;
    return (int)(fit < (size_t)want ? fit : (size_t)want);
}

template <int POLY, int K, int D>
cudaError_t launch_round(const u64* tables, size_t stride, u32 half, const u64* coefs, int eval_one, u64* partials, u32 nblocks, cudaStream_t s) {
    chain_launch(k_sc_round<POLY, K, D>, dim3(nblocks), dim3(RT), 0, s, tables, stride, half, coefs, eval_one, partials);
    return cudaGetLastError();
}

}  // namespace

namespace hlk {

u32 sc_round_blocks(u32 half, int sm_count) {
    u32 b = (half + RT - 1) / RT, cap = (u32)sm_count * 4;
    if (b < 1) b = 1;
    return b > cap ? cap : b;
}

u32 sc_ir_max_blocks(u32 half, int sm_count) {
    u32 b = half, cap = (u32)sm_count * 8;  // the largest grid either form launches
    if (b < 1) b = 1;
    return b > cap ? cap : b;
}

bool sc_ir_fits(const IrDev& p, int degree) { return !ir_pair_capable(p) || ir_pair_warps(p, degree, 1) >= 1; }

u32 sc_ir_blocks(const IrDev& p, u32 half, int degree, int sm_count) {
    u32 per = IRT, cap = (u32)sm_count * 2;
    if (ir_pair_form(p, half)) {
        const int w = ir_pair_warps(p, degree, IRC_MAX_WARPS);
        per = (u32)(w > 0 ? w : 1);
        // CTAs per SM by shared memory
        const size_t cta = ir_fixed_bytes(p) + (size_t)per * ir_area_bytes(p, degree);
        const u32 per_sm = (u32)(IR_SMEM_BUDGET / cta);
        cap = (u32)sm_count * (per_sm < 1 ? 1 : per_sm > 4 ? 4 : per_sm);
    } else if (ir_thread_pair_form(p, half)) {
        cap = (u32)sm_count * 8;
    }
    u32 b = (half + per - 1) / per;
    if (b < 1) b = 1;
    return b > cap ? cap : b;
}

// The single-CTA tail pays off only while a round's pairs fit its warps a few times over.  Thread form (polynomials of a few units):
// a round as three launches costs about 20 us whatever its size, a tail round about 12 us plus 3.4 us per (pair, point) item
// and thread; measured over a block's 23 slot sumchecks, tail from 4,096 entries: 15.97 ms, 1,024: 15.16, 512: 15.06, 256: 14.97,
// 128: 15.21.  Pair form: 16 / 32 / 64 / 128 entries gave 15.77 / 15.97 / 15.85 / 16.28 ms (inside the run-to-run spread but the last).
u32 sc_ir_tail_len(const IrDev& p, int degree) {
    (void)degree;
    return ir_pair_capable(p) ? 32u : 256u;
}

cudaError_t sc_round_ir(const IrDev& p, int k, const u64* tables, size_t stride, u32 half, int degree, int eval_one, u64* partials,
                        u32 nblocks, cudaStream_t s) {
    (void)k;
    if (ir_pair_form(p, half)) {
        const int w = ir_pair_warps(p, degree, IRC_MAX_WARPS);
        if (w < 1) return cudaErrorInvalidValue;
        const size_t smem = ir_fixed_bytes(p) + (size_t)w * ir_area_bytes(p, degree);
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(k_sc_round_irc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
        }
        chain_launch(k_sc_round_irc, dim3(nblocks), dim3(w * 32), smem, s, tables, stride, half, p, degree, eval_one, partials);
        return cudaGetLastError();
    }
    if (ir_thread_pair_form(p, half)) {
        if (p.all_points) {
            const bool skip = !eval_one && p.eval_degree >= 1;
#define IRQ(N)                                                                                                             \
    case N:                                                                                                                \
        if (skip) chain_launch(k_sc_round_irq<N, true>, dim3(nblocks), dim3(IRT), ir_fixed_bytes(p), s, tables, stride, half, p, degree, partials); \
        else chain_launch(k_sc_round_irq<N, false>, dim3(nblocks), dim3(IRT), ir_fixed_bytes(p), s, tables, stride, half, p, degree, partials);     \
        break;
            switch (p.eval_degree + 1) { IRQ(1) IRQ(2) IRQ(3) IRQ(4) IRQ(5) IRQ(6) default: return cudaErrorInvalidValue; }
#undef IRQ
            return cudaGetLastError();
        }
        chain_launch(k_sc_round_irp, dim3(nblocks), dim3(IRT), ir_fixed_bytes(p), s, tables, stride, half, p, degree, eval_one, partials);
        return cudaGetLastError();
    }
    dim3 grid(nblocks, p.eval_degree + 1);  // the rows above are extrapolated by the step
    chain_launch(k_sc_round_ir, dim3(grid), dim3(IRT), ir_fixed_bytes(p), s, tables, stride, half, p, degree, eval_one, partials);
    return cudaGetLastError();
}

cudaError_t sc_tail_ir(const IrDev& p, int k, u64* tables, size_t stride, u32 len, int degree, const ScStep& a, int nrounds,
                       int first_has_claim, cudaStream_t s) {
    if (ir_pair_capable(p)) {
        const int w = ir_pair_warps(p, degree, IR_TAIL_T / 32);
        if (w < 1) return cudaErrorInvalidValue;
        const size_t smem = ir_fixed_bytes(p) + (size_t)w * ir_area_bytes(p, degree);
        if (smem > 32 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(k_sc_tail_ir<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
        }
        chain_launch(k_sc_tail_ir<true>, dim3(1), dim3(w * 32), smem, s, tables, stride, len, p, degree, k, a, nrounds, first_has_claim);
    } else {
        chain_launch(k_sc_tail_ir<false>, dim3(1), dim3(IR_TAIL_T), ir_fixed_bytes(p), s, tables, stride, len, p, degree, k, a, nrounds, first_has_claim);
    }
    return cudaGetLastError();
}

bool sc_supported(int poly, int k, int degree) {
    if (poly == POLY_IR) return k >= 1 && k <= (int)ir::MAX_TABLES && degree >= 1 && degree < SC_MAX_POINTS;
    if (poly == POLY_PROD) return k >= 1 && k <= 6 && degree == k;
    if (poly == POLY_ZC || poly == POLY_LOGUP_T) return k == 4 && degree == 3;
    if (poly == POLY_LOGUP_Q) return k == 3 && degree == 3;
    return false;
}

cudaError_t sc_round(int poly, int k, const u64* tables, size_t stride, u32 half, const u64* coefs, int eval_one, u64* partials,
                     u32 nblocks, cudaStream_t s) {
#define R(P, K, D) return launch_round<P, K, D>(tables, stride, half, coefs, eval_one, partials, nblocks, s)
    switch (poly) {
        case POLY_PROD:
            switch (k) {
                case 1: R(POLY_PROD, 1, 1);
                case 2: R(POLY_PROD, 2, 2);
                case 3: R(POLY_PROD, 3, 3);
                case 4: R(POLY_PROD, 4, 4);
                case 5: R(POLY_PROD, 5, 5);
                case 6: R(POLY_PROD, 6, 6);
            }
            break;
        case POLY_ZC: R(POLY_ZC, 4, 3);
        case POLY_LOGUP_Q: R(POLY_LOGUP_Q, 3, 3);
        case POLY_LOGUP_T: R(POLY_LOGUP_T, 4, 3);
    }
#undef R
    return cudaErrorInvalidValue;
}

template <int POLY, int K, int D>
static cudaError_t launch_fold_round(u64* tables, size_t stride, u32 n, const u64* coefs, const ScState* st, int eval_one, u64* partials, u32 nblocks,
                                     cudaStream_t s) {
    chain_launch(k_sc_fold_round<POLY, K, D>, dim3(nblocks), dim3(RT), 0, s, tables, stride, n, coefs, st, eval_one, partials);
    return cudaGetLastError();
}

// fold with the challenge in `st` and the sums of the next round (table length n after the fold) in one pass
cudaError_t sc_fold_round(int poly, int k, u64* tables, size_t stride, u32 n, const u64* coefs, const ScState* st, int eval_one, u64* partials,
                          u32 nblocks, cudaStream_t s) {
#define R(P, K, D) return launch_fold_round<P, K, D>(tables, stride, n, coefs, st, eval_one, partials, nblocks, s)
    switch (poly) {
        case POLY_PROD:
            switch (k) {
                case 1: R(POLY_PROD, 1, 1);
                case 2: R(POLY_PROD, 2, 2);
                case 3: R(POLY_PROD, 3, 3);
                case 4: R(POLY_PROD, 4, 4);
                case 5: R(POLY_PROD, 5, 5);
                case 6: R(POLY_PROD, 6, 6);
            }
            break;
        case POLY_ZC: R(POLY_ZC, 4, 3);
        case POLY_LOGUP_Q: R(POLY_LOGUP_Q, 3, 3);
        case POLY_LOGUP_T: R(POLY_LOGUP_T, 4, 3);
    }
#undef R
    return cudaErrorInvalidValue;
}

template <int POLY, int K, int D>
static cudaError_t launch_tail(u64* tables, size_t stride, u32 len, const u64* coefs, const ScStep& a, int nrounds, int first_has_claim,
                               u64* scratch, cudaStream_t s) {
    chain_launch(k_sc_tail<POLY, K, D>, dim3(1), dim3(TAIL_T), 0, s, tables, stride, len, coefs, a, nrounds, first_has_claim, scratch);
    return cudaGetLastError();
}

cudaError_t sc_tail(int poly, int k, u64* tables, size_t stride, u32 len, const u64* coefs, const ScStep& a, int nrounds,
                    int first_has_claim, u64* scratch, cudaStream_t s) {
#define R(P, K, D) return launch_tail<P, K, D>(tables, stride, len, coefs, a, nrounds, first_has_claim, scratch, s)
    switch (poly) {
        case POLY_PROD:
            switch (k) {
                case 1: R(POLY_PROD, 1, 1);
                case 2: R(POLY_PROD, 2, 2);
                case 3: R(POLY_PROD, 3, 3);
                case 4: R(POLY_PROD, 4, 4);
                case 5: R(POLY_PROD, 5, 5);
                case 6: R(POLY_PROD, 6, 6);
            }
            break;
        case POLY_ZC: R(POLY_ZC, 4, 3);
        case POLY_LOGUP_Q: R(POLY_LOGUP_Q, 3, 3);
        case POLY_LOGUP_T: R(POLY_LOGUP_T, 4, 3);
    }
#undef R
    return cudaErrorInvalidValue;
}

cudaError_t sc_step(const ScStep& a, cudaStream_t s) {
    chain_launch(k_sc_step, dim3(1), dim3(STEP_T), 0, s, a);
    return cudaGetLastError();
}

cudaError_t sc_nonbase_mask(const u64* tables, size_t stride, size_t len, u32 k, u64* d_mask, int sm_count, cudaStream_t s) {
    size_t bx = (len + 255) / 256, cap = (size_t)sm_count * 8 / (k ? k : 1) + 1;
    if (bx > cap) bx = cap;
    k_sc_nonbase<<<dim3((unsigned)bx, k), 256, 0, s>>>(tables, stride, len, d_mask);
    return cudaGetLastError();
}

cudaError_t sc_fold(u64* tables, size_t stride, u32 half, u32 k, const ScState* st, cudaStream_t s) {
    dim3 grid((half + 255) / 256, k);
    chain_launch(k_sc_fold, dim3(grid), dim3(256), 0, s, tables, stride, half, k, st);
    return cudaGetLastError();
}

}  // namespace hlk
