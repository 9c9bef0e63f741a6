// Row encoder of the Ligero commitment: the per-thread work of every phase.
//
// One CTA encodes one row at a time, entirely in shared memory:
//
//   msg[n] --inverse NTT--> coefficients --(hiding pads, coset powers)--> x[nn], zero above n+q
//          --forward NTT of size nn = R n--> codeword[nn]            (pcs.rs:674-693, ntt.rs:60-108)
//
// The size-nn forward transform is never formed as one transform.  Splitting the
// OUTPUT index k' = R k + s (decimation in frequency on the top log2 R bits) gives
// R independent size-n transforms,
//
//   out[R k + s] = sum_{i<n} y_s[i] w_n^{ik},   y_s[i] = w_nn^{i s} sum_t x[i + t n] w_R^{t s},
//
// and the inner sum has at most T = ceil((n+q)/n) non-zero terms because x is zero
// above n + q.  A size-n row (n <= 2^14) is 128 KB and fits one CTA's shared memory;
// the coefficient blocks x[t n .. t n + n) wait in a per-CTA global scratch slot that
// stays in L2 between its write and its R reads.
//
// Field results are canonical words, so any exact algorithm yields the reference's
// bytes; the transforms here are: inverse = decimation in frequency (natural order in,
// bit-reversed positions out), forward = decimation in time (bit-reversed positions
// in, natural order out).  The bit reversal between them is absorbed into shared-
// memory addressing; nothing is ever permuted in memory.
//
// Every function is a "phase": the kernel calls it for its thread, then barriers.
// The same functions compile for the host, where a test runs the threads of a phase
// one after another and compares whole rows with the CPU oracle.
#pragma once
#include "gl_field.cuh"

// scratch reads go to L2 (the writer is another thread of the same CTA, one barrier earlier)
#ifdef __CUDA_ARCH__
#define ENC_LDCG(p) __ldcg(p)
#else
#define ENC_LDCG(p) (*(p))
#endif

namespace enc {

// Shared-memory index swizzle: XOR every higher nibble into the low nibble.  Any access
// in which the 16 lanes of a half-warp differ in four consecutive index bits (at any
// position, in any order, e.g. bit-reversed) then touches 16 distinct 8-byte banks.
GL_HD u32 swz(u32 p) { return p ^ (((p >> 4) ^ (p >> 8) ^ (p >> 12)) & 15u); }

struct RowArgs {
    const u64* data;   // rows x n
    const u64* pads;   // rows x q   (hiding form only)
    const u64* pows;   // nn coset powers h^i (hiding form only)
    const u64* tw_nn;  // nn powers of the primitive nn-th root w_nn^j
    u64* enc;          // rows x nn
    u64* scratch;      // per CTA: T x n words
    u32 rows, q, T, logr;
    int zk;
    u64 ninv;          // n^-1
};

// ---------------------------------------------------------------------------------------------
// Generic path: radix-2 stages straight on shared memory, any n from 2 to 2^14, any thread count.
// ---------------------------------------------------------------------------------------------
struct Generic {
    GL_HD static void load(const RowArgs& a, u32 row, u32 logn, u64* S, u32 tid, u32 nt) {
        u32 n = 1u << logn;
        for (u32 i = tid; i < n; i += nt) S[i] = a.data[(size_t)row * n + i];
    }
    // one inverse stage, len = 2^ln: (u, v) -> (u + v, (u - v) w^-k)
    GL_HD static void dif_stage(const RowArgs& a, u32 logn, u32 ln, u64* S, u32 tid, u32 nt) {
        u32 n = 1u << logn, nn = n << a.logr, half = 1u << (ln - 1);
        for (u32 b = tid; b < n / 2; b += nt) {
            u32 k = b & (half - 1), i = ((b >> (ln - 1)) << ln) + k;
            u64 u = S[i], v = S[i + half];
            u64 w = a.tw_nn[(nn - ((k << (logn - ln)) << a.logr)) & (nn - 1)];
            S[i] = gl_add(u, v);
            S[i + half] = gl_mul(gl_sub(u, v), w);
        }
    }
    // coefficient blocks x[t n + i], natural order, from the bit-reversed inverse output
    GL_HD static void coeffs(const RowArgs& a, u32 row, u32 logn, const u64* S, u64* X, u32 tid, u32 nt) {
        u32 n = 1u << logn;
        for (u32 i = tid; i < n; i += nt) {
            u64 c = gl_mul(S[gl_brev(i, logn)], a.ninv);
            for (u32 t = 0; t < a.T; t++) {
                u32 idx = i + t * n;
                u64 v = t == 0 ? c : 0;
                if (a.zk) {
                    if (idx < a.q) v = gl_sub(v, a.pads[(size_t)row * a.q + idx]);
                    if (idx >= n && idx - n < a.q) v = gl_add(v, a.pads[(size_t)row * a.q + idx - n]);
                    v = idx < n + a.q ? gl_mul(v, a.pows[idx]) : 0;
                }
                X[(size_t)t * n + i] = v;
            }
        }
    }
    // y_s into shared memory at bit-reversed positions
    GL_HD static void twist(const RowArgs& a, u32 logn, u32 s, const u64* X, u64* S, u32 tid, u32 nt) {
        u32 n = 1u << logn, nn = n << a.logr;
        for (u32 i = tid; i < n; i += nt) {
            u64 y = ENC_LDCG(X + i);
            for (u32 t = 1; t < a.T; t++) y = gl_add(y, gl_mul(ENC_LDCG(X + (size_t)t * n + i), a.tw_nn[(t * s * n) & (nn - 1)]));
            if (s) y = gl_mul(y, a.tw_nn[(i * s) & (nn - 1)]);
            S[gl_brev(i, logn)] = y;
        }
    }
    // one forward stage, len = 2^ln: (u, v) -> (u + v w^k, u - v w^k)
    GL_HD static void dit_stage(const RowArgs& a, u32 logn, u32 ln, u64* S, u32 tid, u32 nt) {
        u32 n = 1u << logn, half = 1u << (ln - 1);
        for (u32 b = tid; b < n / 2; b += nt) {
            u32 k = b & (half - 1), i = ((b >> (ln - 1)) << ln) + k;
            u64 u = S[i], v = gl_mul(S[i + half], a.tw_nn[(k << (logn - ln)) << a.logr]);
            S[i] = gl_add(u, v);
            S[i + half] = gl_sub(u, v);
        }
    }
    GL_HD static void store(const RowArgs& a, u32 row, u32 logn, u32 s, const u64* S, u32 tid, u32 nt) {
        u32 n = 1u << logn;
        size_t nn = (size_t)n << a.logr;
        for (u32 k = tid; k < n; k += nt) a.enc[(size_t)row * nn + ((size_t)k << a.logr) + s] = S[k];
    }
};

// ---------------------------------------------------------------------------------------------
// Fast path, 2^8 <= n <= 2^14: sixteen elements per thread per pass, four stages per pass in
// registers, swizzled shared memory, twiddles w_n^j (j <= n/2) in shared memory.
// ---------------------------------------------------------------------------------------------
template <int LOGN>
struct Fast {
    static constexpr u32 N = 1u << LOGN;
    static constexpr u32 GROUPS = N / 16;   // 16-element groups per pass
    static constexpr u32 TW_WORDS = N / 2 + 16;

    // TW[swz(j)] = w_n^j for j <= n/2 (entry n/2 is -1, so that w^-k = -w^(n/2-k) needs no branch)
    GL_HD static void load_twiddles(const RowArgs& a, u64* TW, u32 tid, u32 nt) {
        for (u32 j = tid; j <= N / 2; j += nt) TW[swz(j)] = j == N / 2 ? GL_P - 1 : a.tw_nn[(size_t)j << a.logr];
    }

    GL_HD static void load(const RowArgs& a, u32 row, u64* S, u32 tid, u32 nt) {
        const u64* src = a.data + (size_t)row * N;
        for (u32 i = tid; i < N; i += nt) S[swz(i)] = src[i];
    }

    // A pass works on the 4-bit window [W, W+4) of the position index: the thread's 16 elements
    // sit at base + j 2^W.  Of the window's bits, only stages LO+1 .. HI (1-based, stage st pairs
    // positions that differ in bit st-1) are executed; W <= LO and HI <= W + 4.
    template <int W>
    GL_HD static u32 group_base(u32 g) { return ((g >> W) << (W + 4)) | (g & ((1u << W) - 1u)); }

    template <int W, int LO, int HI>
    GL_HD static void dit_pass(u64* S, const u64* TW, u32 tid, u32 nt) {
        for (u32 g = tid; g < GROUPS; g += nt) {
            u32 base = group_base<W>(g), k0 = base & ((1u << W) - 1u);
            u64 e[16];
#pragma unroll
            for (int j = 0; j < 16; j++) e[j] = S[swz(base + ((u32)j << W))];
#pragma unroll
            for (int st = LO + 1; st <= HI; st++) {
                const int lb = st - 1 - W;  // bit of j this stage pairs
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (j & (1 << lb)) continue;
                    u32 k = k0 + (((u32)j & ((1u << lb) - 1u)) << W);
                    u64 w = TW[swz(k << (LOGN - st))];
                    u64 u = e[j], v = gl_canon_fast(gl_mul_lazy(e[j | (1 << lb)], w));
                    e[j] = gl_add_lazy(u, v);
                    e[j | (1 << lb)] = gl_sub_lazy(u, v);
                }
            }
#pragma unroll
            for (int j = 0; j < 16; j++) S[swz(base + ((u32)j << W))] = e[j];
        }
    }

    template <int W, int LO, int HI>
    GL_HD static void dif_pass(u64* S, const u64* TW, u32 tid, u32 nt) {
        for (u32 g = tid; g < GROUPS; g += nt) {
            u32 base = group_base<W>(g), k0 = base & ((1u << W) - 1u);
            u64 e[16];
#pragma unroll
            for (int j = 0; j < 16; j++) e[j] = S[swz(base + ((u32)j << W))];
#pragma unroll
            for (int st = HI; st >= LO + 1; st--) {
                const int lb = st - 1 - W;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (j & (1 << lb)) continue;
                    u32 k = k0 + (((u32)j & ((1u << lb) - 1u)) << W);
                    u64 w = GL_P - TW[swz(N / 2 - (k << (LOGN - st)))];  // w^-k = -w^(n/2 - k)
                    u64 u = e[j], v = gl_canon_fast(e[j | (1 << lb)]);
                    e[j] = gl_add_lazy(u, v);
                    e[j | (1 << lb)] = gl_mul_lazy(gl_sub_lazy(u, v), w);
                }
            }
#pragma unroll
            for (int j = 0; j < 16; j++) S[swz(base + ((u32)j << W))] = e[j];
        }
    }

    // the whole transforms as pass lists; `sync` is the barrier between passes
    template <class Sync>
    GL_HD static void inverse(u64* S, const u64* TW, u32 tid, u32 nt, Sync sync) {
        constexpr int R4 = LOGN % 4;
        // windows from the top: [LOGN-4, LOGN), ..., then the remaining low R4 stages in window [0,4)
        if constexpr (LOGN >= 4) { dif_pass<LOGN - 4, LOGN - 4, LOGN>(S, TW, tid, nt); sync(); }
        if constexpr (LOGN >= 8) { dif_pass<LOGN - 8, LOGN - 8, LOGN - 4>(S, TW, tid, nt); sync(); }
        if constexpr (LOGN >= 12) { dif_pass<LOGN - 12, LOGN - 12, LOGN - 8>(S, TW, tid, nt); sync(); }
        if constexpr (R4 > 0) { dif_pass<0, 0, R4>(S, TW, tid, nt); sync(); }
    }
    template <class Sync>
    GL_HD static void forward(u64* S, const u64* TW, u32 tid, u32 nt, Sync sync) {
        constexpr int R4 = LOGN % 4;
        if constexpr (LOGN >= 4) { dit_pass<0, 0, 4>(S, TW, tid, nt); sync(); }
        if constexpr (LOGN >= 8) { dit_pass<4, 4, 8>(S, TW, tid, nt); sync(); }
        if constexpr (LOGN >= 12) { dit_pass<8, 8, 12>(S, TW, tid, nt); sync(); }
        if constexpr (R4 > 0) { dit_pass<LOGN - 4, LOGN - R4, LOGN>(S, TW, tid, nt); sync(); }
    }

    GL_HD static void coeffs(const RowArgs& a, u32 row, const u64* S, u64* X, u32 tid, u32 nt) {
        const u64* pad = a.pads + (size_t)row * a.q;
        for (u32 i = tid; i < N; i += nt) {
            u64 c = gl_mul(S[swz(gl_brev(i, LOGN))], a.ninv);
            for (u32 t = 0; t < a.T; t++) {
                u32 idx = i + t * N;
                u64 v = t == 0 ? c : 0;
                if (a.zk) {
                    if (idx < a.q) v = gl_sub(v, pad[idx]);
                    if (idx >= N && idx - N < a.q) v = gl_add(v, pad[idx - N]);
                    if (idx >= N + a.q) break;
                    v = gl_mul(v, a.pows[idx]);
                }
                X[(size_t)t * N + i] = v;
            }
        }
    }

    GL_HD static void twist(const RowArgs& a, u32 s, const u64* X, u64* S, u32 tid, u32 nt) {
        const u32 nn = N << a.logr;
        for (u32 i = tid; i < N; i += nt) {
            u64 y = ENC_LDCG(X + i);
            // x[i + t n] is zero from i + t n >= n + q on, and those scratch words are never written
            for (u32 t = 1; t < a.T && i + t * N < N + a.q; t++)
                y = gl_add(y, gl_mul(ENC_LDCG(X + (size_t)t * N + i), a.tw_nn[(t * s * N) & (nn - 1)]));
            if (s) y = gl_mul(y, a.tw_nn[(i * s) & (nn - 1)]);
            S[swz(gl_brev(i, LOGN))] = y;
        }
    }

    GL_HD static void store(const RowArgs& a, u32 row, u32 s, const u64* S, u32 tid, u32 nt) {
        u64* dst = a.enc + ((size_t)row * N << a.logr) + s;
        for (u32 k = tid; k < N; k += nt) dst[(size_t)k << a.logr] = gl_canon_fast(S[swz(k)]);  // the passes keep lazy words
    }
};

}  // namespace enc
