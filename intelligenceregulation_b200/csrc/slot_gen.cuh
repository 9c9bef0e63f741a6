// Run-time support of the GENERATED slot kernels: one compiled round kernel per known slot expression graph, the CUDA
// counterpart of the reference's per-slot generated Metal kernels (hashline/src/private_block/metal_slot.rs:115-497,
// `msl_round_kernels`, `gen_kernel`).  The generator (slotgen.py) turns a graph of private_block/slot_ir.rs:57-345 into
// straight-line code in which
//   * every value has a static type, base field or extension field, so no product tests its operands;
//   * a sum of products is accumulated unreduced in 192 bits and reduced once;
//   * table values are loaded where they are first used, so the live set is what the compiler can keep in registers.
// A graph the generator has not seen runs through the interpreter (slot_ir.cuh); both return the reference's words,
// because field arithmetic is exact and the results are canonical.
#pragma once
#include "gl_field.cuh"

namespace sg {

// ---- 192-bit accumulator of 64 x 64-bit products (up to 2^64 of them) ----
struct Acc {
    u64 w0, w1, w2;
};
__device__ __forceinline__ Acc acc_zero() { return Acc{0, 0, 0}; }
__device__ __forceinline__ void mac(Acc& a, u64 x, u64 y) {
    const gl_wide p = gl_mulw(x, y);
    asm("add.cc.u64 %0, %0, %3;\n\taddc.cc.u64 %1, %1, %4;\n\taddc.u64 %2, %2, 0;" : "+l"(a.w0), "+l"(a.w1), "+l"(a.w2) : "l"(p.lo), "l"(p.hi));
}
__device__ __forceinline__ void addw(Acc& a, u64 x) {
    asm("add.cc.u64 %0, %0, %3;\n\taddc.cc.u64 %1, %1, 0;\n\taddc.u64 %2, %2, 0;" : "+l"(a.w0), "+l"(a.w1), "+l"(a.w2) : "l"(x));
}
// w0 + 2^64 (w1 + 2^64 w2) mod p, canonical
__device__ __forceinline__ u64 red(const Acc& a) { return gl_reduce128(a.w0, gl_reduce128(a.w1, a.w2)); }

// ---- an extension-field sum of products: c0 = a0 + 7 a7, c1 = a1 (u^2 = 7, field.rs:163-169) ----
struct AccE {
    Acc a0, a7, a1;
};
__device__ __forceinline__ AccE acce_zero() { return AccE{acc_zero(), acc_zero(), acc_zero()}; }
__device__ __forceinline__ void mac_ee(AccE& a, fp2 x, fp2 y) {
    mac(a.a0, x.c0, y.c0);
    mac(a.a7, x.c1, y.c1);
    mac(a.a1, x.c0, y.c1);
    mac(a.a1, x.c1, y.c0);
}
__device__ __forceinline__ void mac_eb(AccE& a, fp2 x, u64 y) {
    mac(a.a0, x.c0, y);
    mac(a.a1, x.c1, y);
}
__device__ __forceinline__ void mac_bb(AccE& a, u64 x, u64 y) { mac(a.a0, x, y); }
__device__ __forceinline__ void add_e(AccE& a, fp2 x) {
    addw(a.a0, x.c0);
    addw(a.a1, x.c1);
}
__device__ __forceinline__ void add_b(AccE& a, u64 x) { addw(a.a0, x); }
// USED7: some extension x extension product went in
template <bool USED7>
static __device__ __noinline__ fp2 red_e(AccE& a) {
    if constexpr (USED7) mac(a.a0, red(a.a7), 7);
    return f2(red(a.a0), red(a.a1));
}

// A scheduling fence between the nodes of a generated evaluation: without it the compiler hoists every table load of a
// 60-table graph to the top of the function and spills kilobytes; with it a node's loads stay next to their use.
__device__ __forceinline__ void fence() { asm volatile("" ::: "memory"); }

// ---- reduced products for chains of factors ----
__device__ __forceinline__ u64 mul_bb(u64 x, u64 y) { return gl_mul(x, y); }
__device__ __forceinline__ fp2 mul_eb(fp2 x, u64 y) { return f2_mul_base(x, y); }
static __device__ __noinline__ fp2 mul_ee(fp2 x, fp2 y) { return f2_mul(x, y); }
__device__ __forceinline__ u64 neg_b(u64 x) { return gl_neg(x); }
__device__ __forceinline__ fp2 neg_e(fp2 x) { return f2_neg(x); }

// ---- a table's value at evaluation point p of the round's variable: T(i) + p (T(i + half) - T(i)) ----
// p is the same for every thread of a warp.  A base-valued table keeps a zero second word until the first fold, and
// only its first word is read.
static __device__ __noinline__ u64 ld_b(const u64* __restrict__ tb, u32 i, u32 half, u32 p) {
    const u64 lo = tb[2 * (size_t)i];
    if (p == 0) return lo;
    const u64 hi = tb[2 * ((size_t)i + half)];
    if (p == 1) return hi;
    return gl_add(lo, gl_mul(gl_sub(hi, lo), (u64)p));
}
static __device__ __noinline__ fp2 ld_e(const u64* __restrict__ tb, u32 i, u32 half, u32 p) {
    const ulonglong2 a = *reinterpret_cast<const ulonglong2*>(tb + 2 * (size_t)i);
    if (p == 0) return f2(a.x, a.y);
    const ulonglong2 b = *reinterpret_cast<const ulonglong2*>(tb + 2 * ((size_t)i + half));
    if (p == 1) return f2(b.x, b.y);
    return f2(gl_add(a.x, gl_mul(gl_sub(b.x, a.x), (u64)p)), gl_add(a.y, gl_mul(gl_sub(b.y, a.y), (u64)p)));
}

__device__ __forceinline__ u64 shfl_down_u64(u64 v, int d) {
    u32 lo = __shfl_down_sync(0xffffffffu, (u32)v, d), hi = __shfl_down_sync(0xffffffffu, (u32)(v >> 32), d);
    return ((u64)hi << 32) | lo;
}

constexpr int GT = 128;      // threads of a generated round CTA
constexpr int MAX_POINTS = 8;

// One round of a generated graph G.  Evaluated points: j = 0 .. npe - 1 stands for the point j, or j + 1 from j = 1 on when
// the point 1 is skipped (it follows from the running claim).  partials[block][point] as the interpreter's kernels write them.
//   PER_POINT false: a thread takes a pair and walks the points (the tables' words come back from L1 for the later points);
//   PER_POINT true:  a CTA row per point (blockIdx.y), for rounds with fewer pairs than the machine has threads.
template <class G, bool R0, bool PER_POINT>
__global__ void __launch_bounds__(GT, 4) k_slot_round(const u64* __restrict__ tables, size_t stride, u32 half, const u64* __restrict__ cfo, u32 n_cfo,
                                                   int degree, u32 npe, u32 skip_one, u64* __restrict__ partials) {
    extern __shared__ __align__(16) u64 sg_smem[];
    __shared__ u64 wsum[GT / 32][2 * MAX_POINTS];
    fp2* cf = reinterpret_cast<fp2*>(sg_smem);
    for (u32 x = threadIdx.x; x < 2 * n_cfo; x += GT) sg_smem[x] = cfo[x];
    __syncthreads();
    const int np = degree + 1;
    fp2 acc[MAX_POINTS];
#pragma unroll
    for (int d = 0; d < MAX_POINTS; d++) acc[d] = f2(0, 0);
    if constexpr (PER_POINT) {
        const u32 j = blockIdx.y, p = (skip_one && j >= 1) ? j + 1 : j;
        fp2 a = f2(0, 0);
        for (u32 i = blockIdx.x * GT + threadIdx.x; i < half; i += gridDim.x * GT) a = f2_add(a, G::template eval<R0>(tables, stride, i, half, p, cf));
        acc[0] = a;
    } else {
        for (u32 i = blockIdx.x * GT + threadIdx.x; i < half; i += gridDim.x * GT) {
#pragma unroll 1
            for (u32 j = 0; j < npe; j++) {
                const u32 p = (skip_one && j >= 1) ? j + 1 : j;
                acc[j] = f2_add(acc[j], G::template eval<R0>(tables, stride, i, half, p, cf));
            }
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const u32 nacc = PER_POINT ? 1u : npe;
    for (u32 j = 0; j < nacc; j++) {
        fp2 v = acc[j];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            v.c0 = gl_add(v.c0, shfl_down_u64(v.c0, off));
            v.c1 = gl_add(v.c1, shfl_down_u64(v.c1, off));
        }
        if (lane == 0) { wsum[warp][2 * j] = v.c0; wsum[warp][2 * j + 1] = v.c1; }
    }
    __syncthreads();
    if (PER_POINT) {
        const u32 j = blockIdx.y, p = (skip_one && j >= 1) ? j + 1 : j;
        u64* dst = partials + ((size_t)blockIdx.x * np + p) * 2;
        if (threadIdx.x < 2) {
            u64 s = 0;
#pragma unroll
            for (int w = 0; w < GT / 32; w++) s = gl_add(s, wsum[w][threadIdx.x]);
            dst[threadIdx.x] = s;
        }
        if (skip_one && j == 0 && threadIdx.x < 2) partials[((size_t)blockIdx.x * np + 1) * 2 + threadIdx.x] = 0;
    } else if ((int)threadIdx.x < 2 * np) {
        // word x of the CTA's partial row belongs to point d = x / 2: evaluated as acc index j, or zero
        const u32 d = threadIdx.x >> 1, c = threadIdx.x & 1;
        u32 j = d;
        bool live = d < (skip_one ? npe + 1 : npe);
        if (skip_one) { live = live && d != 1; j = d >= 2 ? d - 1 : d; }
        u64 s = 0;
        if (live) {
#pragma unroll
            for (int w = 0; w < GT / 32; w++) s = gl_add(s, wsum[w][2 * j + c]);
        }
        partials[(size_t)blockIdx.x * 2 * np + threadIdx.x] = s;
    }
}

// What the dispatcher knows about a generated graph.
struct Entry {
    u64 signature;       // structural hash of the word stream with every coefficient replaced by its class
    u32 n_tables, n_cfo; // n_cfo: coefficient words of the stream, in order (the kernels index coefficients by occurrence)
    u64 base_mask;       // tables the first-round variant reads as base-valued (bit t)
    const char* name;
    // round launcher: r0 selects the first-round typing, per_point the CTA-row-per-point form
    cudaError_t (*launch)(bool r0, bool per_point, unsigned bx, const u64* tables, size_t stride, u32 half, const u64* cfo, int degree, u32 npe,
                          u32 skip_one, u64* partials, cudaStream_t s);
};

template <class G>
cudaError_t launch_graph(bool r0, bool per_point, unsigned bx, const u64* tables, size_t stride, u32 half, const u64* cfo, int degree, u32 npe,
                         u32 skip_one, u64* partials, cudaStream_t s) {
    const size_t smem = (size_t)G::N_CFO * 16 + 16;
    const dim3 grid(bx, per_point ? npe : 1u);
#define SG_GO(R0, PP) k_slot_round<G, R0, PP><<<grid, GT, smem, s>>>(tables, stride, half, cfo, G::N_CFO, degree, npe, skip_one, partials)
    bool done = false;
    if constexpr (G::HAS_R0) {
        if (r0) {
            if (per_point) SG_GO(true, true); else SG_GO(true, false);
            done = true;
        }
    }
    if (!done) {
        if (per_point) SG_GO(false, true); else SG_GO(false, false);
    }
#undef SG_GO
    return cudaGetLastError();
}

const Entry* find(u64 signature);   // slot_gen_table.cu (generated): NULL for a graph without a generated kernel

}  // namespace sg
