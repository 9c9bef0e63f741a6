// A slot's sumcheck tables built where they are used (private_block/argument.rs:907 build_tables_device; the reference's
// Metal form: gpu/metal.rs MetalTables::{new, plan_eq, plan_plane, build_planned, flush, to_vecs}).
//
// Two table kinds are written by kernels, from small host-made maps, instead of being built on the host and uploaded
// (the 8B block's tables are 1.3 GB per block):
//
//   eq cube      out[x] = hi[y >> p_lo] * lo[y & (2^p_lo - 1)],  y = (x >> shift) & (2^p - 1)
//                with hi, lo the eq tables of the two halves of the point (argument.rs:643-660 eq_cube_split_into);
//   plane        out[x] = sum_z eqf[z] * v(inv(x & used) | zbits[z]),   v(idx) = sum_s coef_s * rows[off_s + idx]
//                a committed witness plane read through the inverse of its index bit map, partially evaluated at the
//                plane's fixed coordinates (argument.rs:386-577 priv_table_fill; the per-output form of :470-540).
//                The rows are the commitment's own resident copy (gpu/metal.rs:3105 MetalCommit::resident_rows).
//
// Every word is the canonical representative of the element the host builder writes: same formula, exact arithmetic,
// only the order of exact additions differs.  A table the caller declares base-valued is checked as it is written
// (imaginary word zero); a violation surfaces at flush as HL_B200_ERR_MISMATCH (metal.rs:2649-2665 refuses the same way).
#include <cstring>
#include <vector>

#include "api_internal.h"
#include "gl_field.cuh"

using namespace hlapi;

// One planned table: what the kernel needs to write it, with its maps as offsets into the two pools of the set's plan.
struct TabDesc {
    u32 kind, table;           // 0 eq cube, 1 plane; the table it fills
    u32 shift, p, p_lo;        // eq
    u32 xlo, nz, ns;           // plane
    int one_slice, base_check;
    u64 used;
    u64 off_a, off_b;          // 64-bit pool: eq hi / lo, or plane eqf / slices
    u64 off_lo, off_hi, off_zb;  // 32-bit pool: plane inv_lo / inv_hi / zbits
    const u64* rows;           // plane: the committed data, flat
    const hl_store* store;     // plane: the commitment those rows belong to, or NULL for caller-owned device rows (host use only)
};

// The eq and plane calls only PLAN a table (MetalTables::plan_eq / plan_plane do the same, gpu/metal.rs): the maps are copied
// into the set's host pools at once, so the caller's arrays are free when the call returns, and everything planned is written by
// one upload and one launch when the set is flushed, read or handed to an evaluator (MetalTables::build_planned).  A slot with
// sixty small tables was sixty launches and some two hundred small copies before.
struct hl_tables {
    hl_ctx* ctx = nullptr;
    u32 k = 0, n_vars = 0;
    u64* d_tables = nullptr;   // k x 2^n_vars Fp2, table-major
    u32* d_flag = nullptr;
    std::vector<TabDesc> plan;
    std::vector<u64> pool64;
    std::vector<u32> pool32;
    size_t len() const { return (size_t)1 << n_vars; }
    size_t bytes() const { return (size_t)k * len() * 16; }
};

namespace {

__device__ __forceinline__ fp2 ld2(const u64* p) {
    ulonglong2 v = *reinterpret_cast<const ulonglong2*>(p);
    return f2(v.x, v.y);
}
__device__ __forceinline__ void st2(u64* p, fp2 v) { *reinterpret_cast<ulonglong2*>(p) = make_ulonglong2(v.c0, v.c1); }

struct PlaneArgs {
    const u64* rows;       // the committed data, flat
    const u32 *inv_lo, *inv_hi, *zbits;
    const u64* eqf;        // nz Fp2 (unused when nz == 0)
    const u64* slices;     // ns x (offset, c0, c1)
    u64 used;
    u32 xlo, nz, ns;
    int one_slice;         // one slice with coefficient 1
    int base_check;
};

__device__ __forceinline__ fp2 plane_value(const PlaneArgs& a, size_t idx) {
    if (a.one_slice) return f2(a.rows[a.slices[0] + idx], 0);
    fp2 v = f2(0, 0);
    for (u32 s = 0; s < a.ns; s++) {
        const u64* sl = a.slices + 3 * (size_t)s;
        v = f2_add(v, f2_mul_base(f2(sl[1], sl[2]), a.rows[sl[0] + idx]));
    }
    return v;
}

__device__ __forceinline__ fp2 plane_entry(const PlaneArgs& a, size_t x) {
    const u64 xu = x & a.used;
    const size_t im = (size_t)a.inv_hi[xu >> a.xlo] | a.inv_lo[xu & (((u64)1 << a.xlo) - 1)];
    if (a.nz == 0) return plane_value(a, im);
    if (a.one_slice) {
        // sum_z eqf[z] * word: the products are summed as integers and reduced once per component
        // (argument.rs:349-384 does the same on the host); 2^128 = -2^32 (mod p) per wrap
        u64 lo0 = 0, hi0 = 0, w0 = 0, lo1 = 0, hi1 = 0, w1 = 0;
        for (u32 z = 0; z < a.nz; z++) {
            const fp2 e = ld2(a.eqf + 2 * (size_t)z);
            const u64 d = a.rows[a.slices[0] + (im | a.zbits[z])];
            const gl_wide p0 = gl_mulw(e.c0, d), p1 = gl_mulw(e.c1, d);
            u64 t = lo0 + p0.lo, c = t < lo0; lo0 = t;
            t = hi0 + p0.hi; u64 c2 = t < hi0; hi0 = t + c; c2 += hi0 < t; w0 += c2;
            t = lo1 + p1.lo; c = t < lo1; lo1 = t;
            t = hi1 + p1.hi; c2 = t < hi1; hi1 = t + c; c2 += hi1 < t; w1 += c2;
        }
        const u64 two128 = 0xFFFFFFFE00000001ull;  // 2^128 mod p
        return f2(gl_add(gl_reduce128(lo0, hi0), gl_mul(w0, two128)), gl_add(gl_reduce128(lo1, hi1), gl_mul(w1, two128)));
    }
    fp2 v = f2(0, 0);
    for (u32 z = 0; z < a.nz; z++) v = f2_add(v, f2_mul(ld2(a.eqf + 2 * (size_t)z), plane_value(a, im | a.zbits[z])));
    return v;
}

// every planned table of a set in one launch: blockIdx.y = the plan entry, blockIdx.x over the table's entries
__global__ void __launch_bounds__(256) k_tab_batch(u64* __restrict__ tables, size_t len, const TabDesc* __restrict__ descs, const u64* __restrict__ p64,
                                                   const u32* __restrict__ p32, u32* __restrict__ flag) {
    __shared__ TabDesc d;
    if (threadIdx.x == 0) d = descs[blockIdx.y];
    __syncthreads();
    const size_t x = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (x >= len) return;
    fp2 v;
    if (d.kind == 0) {
        const size_t y = (x >> d.shift) & (((size_t)1 << d.p) - 1);
        v = f2_mul(ld2(p64 + d.off_a + 2 * (y >> d.p_lo)), ld2(p64 + d.off_b + 2 * (y & (((size_t)1 << d.p_lo) - 1))));
    } else {
        PlaneArgs a;
        a.rows = d.rows; a.inv_lo = p32 + d.off_lo; a.inv_hi = p32 + d.off_hi; a.zbits = p32 + d.off_zb; a.eqf = p64 + d.off_a; a.slices = p64 + d.off_b;
        a.used = d.used; a.xlo = d.xlo; a.nz = d.nz; a.ns = d.ns; a.one_slice = d.one_slice; a.base_check = d.base_check;
        v = plane_entry(a, x);
    }
    st2(tables + 2 * ((size_t)d.table * len + x), v);
    if (d.base_check && v.c1 != 0) atomicOr(flag, 1u);
}

// uploads a small host array into a pool allocation; the caller frees it after the launch (stream-ordered)
template <class T>
int upload(hl_ctx* c, const void* h, size_t count, T** d) {
    *d = nullptr;
    if (count == 0) return HL_B200_OK;
    int rc = dev_alloc(c, (void**)d, count * sizeof(T));
    if (!rc) rc = h2d_owned(c, *d, h, count * sizeof(T));
    return rc;
}

}  // namespace

u64* hl_tables_adopt(hl_tables* t) {  // rounds_api.cu takes the device tables over
    u64* p = t->d_tables;
    t->d_tables = nullptr;
    return p;
}

const u64* hl_tables_peek(hl_tables* t) { return t->d_tables; }

void hl_tables_shape(hl_tables* t, hl_ctx** c, size_t* k, uint32_t* n_vars) {
    *c = t->ctx;
    *k = t->d_tables ? t->k : 0;
    *n_vars = t->n_vars;
}

// writes every planned table: one upload of the descriptors and the two pools, one launch; the caller holds the context's lock
static int launch_planned(hl_tables* t) {
    if (t->plan.empty()) return HL_B200_OK;
    hl_ctx* c = t->ctx;
    for (const TabDesc& d : t->plan)
        if (d.kind == 1 && d.store && !c->stores.count(d.store)) {  // the rows are gone: nothing is launched over them
            t->plan.clear(); t->pool64.clear(); t->pool32.clear();
            return fail(c, HL_B200_ERR_ARG, "tables: a planned plane's commitment was freed before the set was built");
        }
    TabDesc* d_desc = nullptr;
    u64* d_p64 = nullptr;
    u32* d_p32 = nullptr;
    const size_t nd = t->plan.size(), n64 = t->pool64.size(), n32 = t->pool32.size();
    int rc;
    {
        Timed tm(c, HL_T_TABLES);  // the span takes the maps' upload with it: it is part of what building the tables costs
        rc = upload(c, t->plan.data(), nd, &d_desc);
        if (!rc) rc = upload(c, t->pool64.data(), n64, &d_p64);
        if (!rc) rc = upload(c, t->pool32.data(), n32, &d_p32);
        if (!rc) {
            const size_t len = t->len();
            k_tab_batch<<<dim3((unsigned)((len + 255) / 256), (unsigned)nd), 256, 0, c->stream>>>(t->d_tables, len, d_desc, d_p64, d_p32, t->d_flag);
            c->stats.kernel_launches++;
            cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "planned tables launch", e);
        }
    }
    if (d_desc) dev_free(c, d_desc, nd * sizeof(TabDesc));
    if (d_p64) dev_free(c, d_p64, n64 * 8);
    if (d_p32) dev_free(c, d_p32, n32 * 4);
    t->plan.clear();
    t->pool64.clear();
    t->pool32.clear();
    return rc;
}

int hl_tables_flush_locked(hl_tables* t) {
    hl_ctx* c = t->ctx;
    u32 flag = 0;
    int rc = launch_planned(t);
    if (!rc) rc = d2h(c, &flag, t->d_flag, 4);
    if (!rc) rc = sync(c, "tables_flush");
    if (!rc && flag) rc = fail(c, HL_B200_ERR_MISMATCH, "tables: a table declared base-valued holds an extension word");
    return rc;
}

extern "C" {

int hl_b200_tables_new(hl_ctx* c, size_t k, uint32_t n_vars, hl_tables** out) {
    if (!c || !out || k == 0) return fail(c, HL_B200_ERR_ARG, "tables_new: null argument or no table");
    if (n_vars > 30 || k > 64) return fail(c, HL_B200_ERR_UNSUPPORTED, "tables_new: more than 30 variables or 64 tables");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    hl_tables* t = new hl_tables();
    t->ctx = c; t->k = (u32)k; t->n_vars = n_vars;
    int rc = dev_alloc(c, (void**)&t->d_tables, t->bytes());
    if (!rc) rc = dev_alloc(c, (void**)&t->d_flag, 4);
    if (!rc) {
        cudaError_t e = cudaMemsetAsync(t->d_flag, 0, 4, c->stream);
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "tables_new", e);
    }
    if (rc) {
        if (t->d_tables) dev_free(c, t->d_tables, t->bytes());
        if (t->d_flag) dev_free(c, t->d_flag, 4);
        delete t;
        return rc;
    }
    *out = t;
    return HL_B200_OK;
}

void hl_b200_tables_free(hl_tables* t) {
    if (!t) return;
    hl_ctx* c = t->ctx;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    if (t->d_tables) dev_free(c, t->d_tables, t->bytes());
    dev_free(c, t->d_flag, 4);
    delete t;
}

int hl_b200_tables_put(hl_tables* t, size_t i, const uint64_t* words) {
    if (!t || !words || !t->d_tables || i >= t->k) return HL_B200_ERR_ARG;
    hl_ctx* c = t->ctx;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    if (int rc = launch_planned(t)) return rc;  // a planned table may be the one overwritten here: keep the caller's order
    return h2d_owned(c, t->d_tables + 2 * i * t->len(), words, t->len() * 16);
}

int hl_b200_tables_eq(hl_tables* t, size_t i, uint32_t start, uint32_t p, const uint64_t* hi, const uint64_t* lo, int base_check) {
    if (!t || !t->d_tables || i >= t->k || !hi || !lo) return HL_B200_ERR_ARG;
    hl_ctx* c = t->ctx;
    if (start + p > t->n_vars) return fail(c, HL_B200_ERR_ARG, "tables_eq: start + |point| exceeds the cube");  // argument.rs:604-607
    const u32 p_lo = p / 2, shift = t->n_vars - start - p;
    std::lock_guard<std::mutex> g(c->mu);
    const size_t nhi = (size_t)2 << (p - p_lo), nlo = (size_t)2 << p_lo;
    TabDesc d;
    memset(&d, 0, sizeof d);
    d.kind = 0; d.table = (u32)i; d.shift = shift; d.p = p; d.p_lo = p_lo; d.base_check = base_check;
    d.off_a = t->pool64.size();
    t->pool64.insert(t->pool64.end(), hi, hi + nhi);
    d.off_b = t->pool64.size();
    t->pool64.insert(t->pool64.end(), lo, lo + nlo);
    t->plan.push_back(d);
    return HL_B200_OK;
}

int hl_b200_tables_plane(hl_tables* t, size_t i, const hl_store* store, const uint64_t* d_rows, size_t n_words, uint64_t used, uint32_t xlo,
                         const uint32_t* inv_lo, const uint32_t* inv_hi, const uint32_t* zbits, uint32_t nz, const uint64_t* eqf,
                         const uint64_t* slices, uint32_t ns, int base_check) {
    if (!t || !t->d_tables || i >= t->k || !inv_lo || !inv_hi || !slices || ns == 0) return HL_B200_ERR_ARG;
    hl_ctx* c = t->ctx;
    if (store) {
        if (store->ctx != c) return fail(c, HL_B200_ERR_ARG, "tables_plane: the commitment belongs to another context");
        d_rows = reinterpret_cast<const uint64_t*>(store->d_data);
        n_words = (size_t)store->rows * store->n();
    }
    if (!d_rows) return fail(c, HL_B200_ERR_ARG, "tables_plane: no rows");
    if (nz && (!zbits || !eqf)) return fail(c, HL_B200_ERR_ARG, "tables_plane: fixed coordinates without their maps");
    if (xlo > t->n_vars || t->n_vars - xlo > 24 || xlo > 24 || nz > (1u << 16)) return fail(c, HL_B200_ERR_UNSUPPORTED, "tables_plane: map sizes");
    // every address the kernel can form stays inside the rows: the index is an OR of map entries
    const size_t nlo = (size_t)1 << xlo, nhi = (size_t)1 << (t->n_vars - xlo);
    u64 all = 0, max_off = 0;
    for (size_t j = 0; j < nlo; j++) all |= inv_lo[j];
    for (size_t j = 0; j < nhi; j++) all |= inv_hi[j];
    for (u32 z = 0; z < nz; z++) all |= zbits[z];
    for (u32 s = 0; s < ns; s++) max_off = slices[3 * (size_t)s] > max_off ? slices[3 * (size_t)s] : max_off;
    if (max_off >= n_words || all >= n_words - max_off) return fail(c, HL_B200_ERR_ARG, "tables_plane: a slice reaches past the committed rows");
    std::lock_guard<std::mutex> g(c->mu);
    TabDesc d;
    memset(&d, 0, sizeof d);
    d.kind = 1; d.table = (u32)i; d.xlo = xlo; d.nz = nz; d.ns = ns; d.used = used; d.base_check = base_check;
    d.one_slice = ns == 1 && slices[1] == 1 && slices[2] == 0;
    d.rows = reinterpret_cast<const u64*>(d_rows);
    d.store = store;
    d.off_lo = t->pool32.size();
    t->pool32.insert(t->pool32.end(), inv_lo, inv_lo + nlo);
    d.off_hi = t->pool32.size();
    t->pool32.insert(t->pool32.end(), inv_hi, inv_hi + nhi);
    d.off_zb = t->pool32.size();
    if (nz) t->pool32.insert(t->pool32.end(), zbits, zbits + nz);
    d.off_a = t->pool64.size();  // even: every 64-bit array read as Fp2 starts on a 16-byte boundary
    if (nz) t->pool64.insert(t->pool64.end(), eqf, eqf + (size_t)nz * 2);
    d.off_b = t->pool64.size();
    t->pool64.insert(t->pool64.end(), slices, slices + (size_t)ns * 3);
    if (t->pool64.size() & 1) t->pool64.push_back(0);
    t->plan.push_back(d);
    return HL_B200_OK;
}

int hl_b200_tables_flush(hl_tables* t) {
    if (!t || !t->d_tables) return HL_B200_ERR_ARG;
    hl_ctx* c = t->ctx;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    return hl_tables_flush_locked(t);
}

int hl_b200_tables_read(hl_tables* t, size_t i, uint64_t* out) {
    if (!t || !t->d_tables || i >= t->k || !out) return HL_B200_ERR_ARG;
    hl_ctx* c = t->ctx;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    int rc = launch_planned(t);
    if (!rc) rc = d2h(c, out, t->d_tables + 2 * i * t->len(), t->len() * 16);
    if (!rc) rc = sync(c, "tables_read");
    return rc;
}

}  // extern "C"
