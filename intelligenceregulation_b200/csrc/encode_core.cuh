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

// one packed witness word widened to its canonical field word
GL_HD u64 widen_word(const unsigned char* base, u32 i, u32 w) {
    long long x;
    if (w == 1) x = (long long)reinterpret_cast<const signed char*>(base)[i];
    else if (w == 2) x = (long long)reinterpret_cast<const short*>(base)[i];
    else if (w == 4) x = (long long)reinterpret_cast<const int*>(base)[i];
    else return reinterpret_cast<const u64*>(base)[i];
    return x >= 0 ? (u64)x : GL_P - (u64)(-x);
}

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
    u64* scratch;      // per CTA: T x N words, N = the size the shared-memory transforms run at
    u32 rows, q;
    u32 T;             // coefficient blocks of N words: ceil((n + q) / N) (hiding form) or n / N (plain form)
    u32 logr;          // log2(nn / N): the number of output residues
    u32 loga;          // log2(n / N): 0 unless the row is longer than one shared-memory transform
    int zk;
    u64 ninv;          // n^-1
    u64* coef_out;     // FORM_COSET only: the row's n coefficients, in rows of 2n words (or NULL)
    // packed witness rows (fast path, FORM_PCS): row r is `row_w[r]`-byte two's-complement little-endian integers (1, 2, 4; 8 =
    // the canonical word itself) starting at byte `row_off[r]` of `narrow`; the first pass widens them (x >= 0 -> x, x < 0 ->
    // p + x, field.rs:32-34) and leaves the 64-bit row in `data`, which the opening folds read later.  NULL: `data` is the input.
    const unsigned char* narrow = nullptr;
    const u64* row_off = nullptr;
    const unsigned char* row_w = nullptr;
    int split;         // fast path: a CTA takes one (row, output residue) instead of a whole row, repeating the row's inverse transform:
                       // for a handful of rows (fewer than SMs / residues) the latency of a row falls from 1 + R transforms to 2
};

// What a row is and how its coefficients are twisted (template argument of Fast::row_coeffs).
//   FORM_PCS    the commitment forms above: plain (no twist) or hiding (pads folded in, coset powers)
//   FORM_COSET  n evaluations -> n coefficients c, x[i] = c[i] h^i, c kept in coef_out (a masking commitment's message rows,
//               hashline/src/zk.rs:463-476: pads sit inside the message, the coset is applied to every row)
//   FORM_COEF   n + q coefficients given as such, x[i] = c[i] h^i (its blinding and proximity rows, zk.rs:478-487)
enum { FORM_PCS = 0, FORM_COSET = 1, FORM_COEF = 2 };

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
// registers, swizzled shared memory, twiddles w_n^j (j < n/2) in shared memory.
//
// Both directions run the SAME forward decimation-in-time passes: the inverse transform of msg is
// c[i] = X[(n - i) mod n] / n with X the forward transform of msg, so the coefficient step just
// reads the forward output at the negated index.  A transform is
//     first pass   source(i) -> registers (16 values of stride n/16, coalesced over the lanes)
//                  -> stages 1..4 -> shared memory at bit-reversed positions
//     middle       shared -> stages -> shared, one 4-bit window of the position index per pass
//     last pass    shared -> the remaining stages -> sink(k, value) straight from registers
// so a row's words cross shared memory (passes - 1) times, and neither the input permutation nor
// the output store is a pass of its own.  Words are "lazy" (any u64 congruent mod p) between passes;
// the sinks canonicalise.
// ---------------------------------------------------------------------------------------------
template <int LOGN>
struct Fast {
    static_assert(LOGN >= 8 && LOGN <= 14, "fast path sizes");
    static constexpr u32 N = 1u << LOGN;
    static constexpr u32 GROUPS = N / 16;   // 16-element groups per pass
    static constexpr u32 TW_WORDS = N / 2;
    static constexpr int R4 = LOGN % 4;
    static constexpr int LASTW = LOGN - 4;  // window of the last pass
    static constexpr int LASTLO = R4 ? LOGN - R4 : LOGN - 4;

    // swz is linear over XOR, so swz(base | c) = swz(base) ^ swz(c) whenever base and c share no bit:
    // one swizzle per group, compile-time constants per element.
    static GL_HDC u32 swzc(u32 p) { return p ^ (((p >> 4) ^ (p >> 8) ^ (p >> 12)) & 15u); }
    static GL_HDC u32 brev4(u32 j) { return ((j & 1) << 3) | ((j & 2) << 1) | ((j & 4) >> 1) | ((j & 8) >> 3); }

    // TW[swz(j)] = w_n^j, j < n/2
    GL_HD static void load_twiddles(const RowArgs& a, u64* TW, u32 tid, u32 nt) {
        for (u32 j = tid; j < N / 2; j += nt) TW[swz(j)] = a.tw_nn[(size_t)j << a.logr];
    }

    template <int W>
    GL_HD static u32 group_base(u32 g) { return ((g >> W) << (W + 4)) | (g & ((1u << W) - 1u)); }

    // Stages LO+1 .. HI (1-based; stage st pairs positions that differ in bit st-1) on the 16 elements of the
    // window [W, W+4); k0 = the group's position bits below the window.  Lazy in, lazy out.
    template <int W, int LO, int HI>
    GL_HD static void stages(u64 (&e)[16], const u64* TW, u32 k0) {
#pragma unroll
        for (int st = LO + 1; st <= HI; st++) {
            const int lb = st - 1 - W;  // bit of j this stage pairs
            const u32 tbase = W > 0 ? swz(k0 << (LOGN - st)) : 0u;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                if (j & (1 << lb)) continue;
                const u32 jm = (u32)j & ((1u << lb) - 1u);
                u64 u = e[j], v;
                if (W == 0 && jm == 0) {
                    v = gl_canon_fast(e[j | (1 << lb)]);  // twiddle 1
                } else {
                    const u64 w = TW[tbase ^ swzc((jm << W) << (LOGN - st))];
                    v = gl_canon_fast(gl_mul_lazy(e[j | (1 << lb)], w));
                }
                e[j] = gl_add_lazy(u, v);
                e[j | (1 << lb)] = gl_sub_lazy(u, v);
            }
        }
    }

    // first pass: element i of the transform's input comes from source(i); lanes take neighbouring i
    template <class Source>
    GL_HD static void first_pass(u64* S, const u64* TW, u32 tid, u32 nt, Source source) {
        for (u32 t = tid; t < GROUPS; t += nt) {
            u64 e[16];
#pragma unroll
            for (int j = 0; j < 16; j++) e[j] = source(t + brev4((u32)j) * GROUPS);  // position 16 g + j holds index brev(16 g + j)
            stages<0, 0, 4>(e, TW, 0);
            const u32 sb = swz(gl_brev(t, LOGN - 4) << 4);
#pragma unroll
            for (int j = 0; j < 16; j++) S[sb ^ swzc((u32)j)] = e[j];
        }
    }

    template <int W>
    GL_HD static void mid_pass(u64* S, const u64* TW, u32 tid, u32 nt) {
        for (u32 g = tid; g < GROUPS; g += nt) {
            const u32 base = group_base<W>(g), sb = swz(base);
            u64 e[16];
#pragma unroll
            for (int j = 0; j < 16; j++) e[j] = S[sb ^ swzc((u32)j << W)];
            stages<W, W, W + 4>(e, TW, base & ((1u << W) - 1u));
#pragma unroll
            for (int j = 0; j < 16; j++) S[sb ^ swzc((u32)j << W)] = e[j];
        }
    }

    // last pass: output k = g + j n/16 goes to sink(k, lazy value)
    template <class Sink>
    GL_HD static void last_pass(const u64* S, const u64* TW, u32 tid, u32 nt, Sink sink) {
        for (u32 g = tid; g < GROUPS; g += nt) {
            const u32 sb = swz(g);
            u64 e[16];
#pragma unroll
            for (int j = 0; j < 16; j++) e[j] = S[sb ^ swzc((u32)j << LASTW)];
            stages<LASTW, LASTLO, LOGN>(e, TW, g);
#pragma unroll
            for (int j = 0; j < 16; j++) sink(g + ((u32)j << LASTW), e[j]);
        }
    }

    template <class Source, class Sink, class Sync>
    GL_HD static void transform(u64* S, const u64* TW, u32 tid, u32 nt, Source source, Sink sink, Sync sync) {
        first_pass(S, TW, tid, nt, source);
        sync();
        // full 4-stage windows below the last pass's first stage: [4,8) when LASTLO >= 8, [8,12) when LASTLO >= 12
        if constexpr (LASTLO >= 8) { mid_pass<4>(S, TW, tid, nt); sync(); }
        if constexpr (LASTLO >= 12) { mid_pass<8>(S, TW, tid, nt); sync(); }
        last_pass(S, TW, tid, nt, sink);
    }

    // ---- the row pipeline ----
    // inverse transform of the message row, then the coefficient blocks x[idx] into the scratch slot.
    // c[i] = F[(n - i) mod n] / n with F the forward transform of the message, one residue a of F per pass set.
    template <class Sync, int FORM = FORM_PCS, bool NARROW = false>
    GL_HD static void row_coeffs(const RowArgs& a, u32 row, u64* S, const u64* TW, u64* X, u32 tid, u32 nt, Sync sync) {
        const u32 A = 1u << a.loga, n = N << a.loga, nn = N << a.logr, lognn = LOGN + a.logr;
        if constexpr (FORM == FORM_COEF) {
            const u64* cs = a.data + (size_t)row * (n + a.q);
            for (u32 i = tid; i < n + a.q; i += nt) X[i] = gl_mul(cs[i], a.pows[i]);
            return;
        }
        const u64* src = a.data + (size_t)row * n;
        const u64* pad = a.pads + (size_t)row * a.q;
        const u32 Tn = a.zk ? (n + a.q + n - 1) / n : 1u;
        const unsigned char* nsrc = nullptr;
        u32 nw = 8;
        if constexpr (NARROW) { nsrc = a.narrow + a.row_off[row]; nw = a.row_w[row]; }
        for (u32 ra = 0; ra < A; ra++) {
            transform(S, TW, tid, nt,
                      [&](u32 i) {
                          u64 y;
                          if constexpr (NARROW) {  // loga == 0 on this path: every word of the row passes here exactly once
                              y = widen_word(nsrc, i, nw);
                              const_cast<u64*>(src)[i] = y;
                          } else {
                              y = src[i];
                          }
                          if (a.loga) {
                              for (u32 t = 1; t < A; t++)
                                  y = gl_add(y, gl_mul_fast(src[i + t * N], a.tw_nn[((t * ra) << (lognn - a.loga)) & (nn - 1)]));  // w_A^(t a)
                              if (ra) y = gl_mul_lazy(y, a.tw_nn[((i * ra) << (a.logr - a.loga)) & (nn - 1)]);                // w_n^(i a); a pass takes lazy words
                          }
                          return y;
                      },
                      [&](u32 k, u64 v) {
                          const u32 i = (n - ((k << a.loga) + ra)) & (n - 1);
                          const u64 c = gl_mul_fast(v, a.ninv);
                          if constexpr (FORM == FORM_COSET) {
                              X[i] = gl_mul(c, a.pows[i]);
                              if (a.coef_out) a.coef_out[(size_t)row * 2 * n + i] = c;
                          } else {
                              for (u32 t = 0; t < Tn; t++) {
                                  const u32 idx = i + t * n;
                                  u64 x = t == 0 ? c : 0;
                                  if (a.zk) {
                                      if (idx >= n + a.q) break;
                                      if (idx < a.q) x = gl_sub(x, pad[idx]);
                                      if (idx >= n && idx - n < a.q) x = gl_add(x, pad[idx - n]);
                                      x = gl_mul_fast(x, a.pows[idx]);
                                  }
                                  X[idx] = x;
                              }
                          }
                      },
                      sync);
            if (ra + 1 < A) sync();  // the next residue's first pass overwrites the shared-memory row
        }
    }

    // output residue s: the size-N transform of the twisted coefficients, stored at out[(nn/N) k + s]
    template <class Sync>
    GL_HD static void row_residue(const RowArgs& a, u32 row, u32 s, u64* S, const u64* TW, const u64* X, u32 tid, u32 nt, Sync sync) {
        const u32 nn = N << a.logr, live = (N << a.loga) + a.q;  // x is zero from n + q on (plain form: q = 0)
        u64* dst = a.enc + ((size_t)row * N << a.logr) + s;
        transform(S, TW, tid, nt,
                  [&](u32 i) {
                      u64 y = ENC_LDCG(X + i);
                      // the scratch words from n + q on are never written and never read
                      for (u32 t = 1; t < a.T && i + t * N < live; t++)
                          y = gl_add(y, gl_mul_fast(ENC_LDCG(X + (size_t)t * N + i), a.tw_nn[(t * s * N) & (nn - 1)]));
                      if (s) y = gl_mul_lazy(y, a.tw_nn[(i * s) & (nn - 1)]);  // a pass takes lazy words
                      return y;
                  },
                  [&](u32 k, u64 v) { dst[(size_t)k << a.logr] = gl_canon_fast(v); }, sync);
    }
};

}  // namespace enc
