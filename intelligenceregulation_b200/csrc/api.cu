// The C ABI of the backend (include/hl_b200.h): context, commitments, stores, Merkle trees.
// Host runtime only; the kernels live in encode.cu, hash.cu, store.cu, misc.cu.
#include "api_internal.h"
#include "../../include/hl_b200_bench.h"

#include <cstdio>
#include <cstring>

using namespace hlapi;

namespace hlapi {

int fail(hl_ctx* c, int code, const char* what, cudaError_t e) {
    if (c) {
        char buf[512];
        if (e != cudaSuccess) snprintf(buf, sizeof buf, "%s: %s", what, cudaGetErrorString(e));
        else snprintf(buf, sizeof buf, "%s", what);
        std::lock_guard<std::mutex> g(c->err_mu);
        c->last_error = buf;
        c->stats.declines++;
    }
    return code;
}

// Stream-ordered allocation from the device's default pool, whose release threshold is
// lifted at init so that freed blocks are reused instead of returned to the driver.
int dev_alloc(hl_ctx* c, void** p, size_t bytes) {
    *p = nullptr;
    if (bytes == 0) bytes = 16;
    if (c->alloc_cap && c->alloc_live + bytes > c->alloc_cap) return fail(c, HL_B200_ERR_OOM, "allocation cap reached (test hook)");
    cudaError_t e = cudaMallocAsync(p, bytes, c->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(c, HL_B200_ERR_OOM, "cudaMallocAsync", e);
    }
    c->alloc_live += bytes;
    return HL_B200_OK;
}

void dev_free(hl_ctx* c, void* p, size_t bytes) {
    if (!p) return;
    cudaFreeAsync(p, c->stream);
    if (bytes == 0) bytes = 16;
    c->alloc_live = c->alloc_live >= bytes ? c->alloc_live - bytes : 0;
}

int h2d(hl_ctx* c, void* d, const void* h, size_t bytes) {
    if (!bytes) return HL_B200_OK;
    cudaError_t e = cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, c->stream);
    if (e != cudaSuccess) return fail(c, HL_B200_ERR_DEVICE, "copy to device", e);
    c->stats.bytes_h2d += bytes;
    return HL_B200_OK;
}

// An asynchronous copy out of page-locked caller memory reads the source when the DMA runs, not when the call is made: a call
// that returns without synchronising would let the caller overwrite inputs that are still to be read.  Small inputs are
// bounced through a page-locked area of the context (reused after a synchronisation when it wraps); large ones are copied
// in place and waited for.
constexpr size_t ARENA_BYTES = (size_t)4 << 20;
int h2d_owned(hl_ctx* c, void* d, const void* h, size_t bytes) {
    if (!bytes) return HL_B200_OK;
    if (!c->arena && cudaHostAlloc((void**)&c->arena, ARENA_BYTES, cudaHostAllocDefault) != cudaSuccess) {
        cudaGetLastError();
        c->arena = nullptr;
    }
    if (c->arena && bytes <= ARENA_BYTES / 4) {
        const size_t need = (bytes + 63) & ~(size_t)63;
        if (c->arena_off + need > ARENA_BYTES) {
            cudaError_t e = cudaStreamSynchronize(c->stream);
            if (e != cudaSuccess) return fail(c, HL_B200_ERR_DEVICE, "staging area", e);
            c->arena_off = 0;
        }
        char* slot = c->arena + c->arena_off;
        c->arena_off += need;
        memcpy(slot, h, bytes);
        return h2d(c, d, slot, bytes);
    }
    int rc = h2d(c, d, h, bytes);
    if (!rc) rc = sync(c, "copy to device");
    return rc;
}

int d2h(hl_ctx* c, void* h, const void* d, size_t bytes) {
    if (!bytes) return HL_B200_OK;
    cudaError_t e = cudaMemcpyAsync(h, d, bytes, cudaMemcpyDeviceToHost, c->stream);
    if (e != cudaSuccess) return fail(c, HL_B200_ERR_DEVICE, "copy from device", e);
    c->stats.bytes_d2h += bytes;
    return HL_B200_OK;
}

int sync(hl_ctx* c, const char* what) {
    cudaError_t e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) return fail(c, HL_B200_ERR_DEVICE, what, e);
    return HL_B200_OK;
}

// w_nn^j for j < nn, w_nn = 7^((p-1)/2^32)^(2^(32-log nn)) (field.rs:86-91, ntt.rs:29-43);
// built once per size on the host and kept on the device.
int root_powers(hl_ctx* c, u32 lognn, const u64** out) {
    auto it = c->tw.find(lognn);
    if (it != c->tw.end()) { *out = it->second; return HL_B200_OK; }
    if (lognn > 26) return fail(c, HL_B200_ERR_UNSUPPORTED, "transform size above 2^26");
    size_t nn = (size_t)1 << lognn;
    std::vector<u64> h(nn);
    u64 r32 = gl_pow(7, (GL_P - 1) >> 32), w = gl_pow(r32, 1ULL << (32 - lognn)), cur = 1;
    for (size_t j = 0; j < nn; j++) { h[j] = cur; cur = gl_mul(cur, w); }
    void* d = nullptr;
    cudaError_t e = cudaMalloc(&d, nn * 8);
    if (e != cudaSuccess) return fail(c, HL_B200_ERR_OOM, "twiddle table", e);
    e = cudaMemcpyAsync(d, h.data(), nn * 8, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);  // h dies at return
    if (e != cudaSuccess) { cudaFree(d); return fail(c, HL_B200_ERR_DEVICE, "twiddle upload", e); }
    c->tw[lognn] = (u64*)d;
    *out = (u64*)d;
    return HL_B200_OK;
}

// a 32-byte key as eight device words; NULL stays NULL (unkeyed)
int upload_key(hl_ctx* c, const uint8_t* key32, uint32_t** d_key) {
    *d_key = nullptr;
    if (!key32) return HL_B200_OK;
    int rc = dev_alloc(c, (void**)d_key, 32);
    if (rc) return rc;
    return h2d_owned(c, *d_key, key32, 32);  // little-endian host: the bytes are the words
}

int log2_exact(size_t v) {
    if (v == 0 || (v & (v - 1))) return -1;
    int l = 0;
    while (((size_t)1 << l) < v) l++;
    return l;
}

static cudaEvent_t take_event(hl_ctx* c) {
    if (!c->ev_pool.empty()) { cudaEvent_t e = c->ev_pool.back(); c->ev_pool.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

Timed::Timed(hl_ctx* ctx, int cls) : c(ctx), on(ctx->timing) {
    if (!on) return;
    s.a = take_event(c); s.b = take_event(c); s.cls = cls;
    cudaEventRecord(s.a, c->stream);
}
Timed::~Timed() {
    if (!on) return;
    cudaEventRecord(s.b, c->stream);
    c->spans.push_back(s);
}

}  // namespace hlapi

extern "C" {

int hl_b200_timing_enable(hl_ctx* c, int on) {
    if (!c) return HL_B200_ERR_ARG;
    std::lock_guard<std::mutex> g(c->mu);
    c->timing = on != 0;
    return HL_B200_OK;
}

int hl_b200_timing_read(hl_ctx* c, hl_timing* out, int reset) {
    if (!c || !out) return HL_B200_ERR_ARG;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    int rc = sync(c, "timing_read");
    if (rc) return rc;
    for (auto& s : c->spans) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, s.a, s.b) == cudaSuccess) { c->timing_acc.ms[s.cls] += ms; c->timing_acc.spans[s.cls]++; }
        c->ev_pool.push_back(s.a); c->ev_pool.push_back(s.b);
    }
    c->spans.clear();
    *out = c->timing_acc;
    if (reset) c->timing_acc = hl_timing{};
    return HL_B200_OK;
}

int hl_b200_init(int device, hl_ctx** out) {
    if (!out) return HL_B200_ERR_ARG;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || device < 0 || device >= count) return HL_B200_ERR_DEVICE;
    if (cudaSetDevice(device) != cudaSuccess) return HL_B200_ERR_DEVICE;
    hl_ctx* c = new hl_ctx();
    c->device = device;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete c; return HL_B200_ERR_DEVICE; }
    c->sm_count = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking) != cudaSuccess) { delete c; return HL_B200_ERR_DEVICE; }
    c->stream = c->own_stream;
    if (cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_main, cudaEventDisableTiming) != cudaSuccess) { delete c; return HL_B200_ERR_DEVICE; }
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
        unsigned long long keep = ~0ULL;
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    char buf[512];
    snprintf(buf, sizeof buf, "hl_b200: %s (sm_%d%d, %d SMs, %.0f GB), device %d", prop.name, prop.major, prop.minor,
             prop.multiProcessorCount, (double)prop.totalGlobalMem / 1e9, device);
    c->label = buf;
    *out = c;
    return HL_B200_OK;
}

void hl_b200_shutdown(hl_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    for (auto& kv : c->tw) cudaFree(kv.second);
    if (c->d_wp_flag) cudaFree(c->d_wp_flag);
    for (int i = 0; i < 2; i++) {
        if (c->stage[i]) cudaFreeHost(c->stage[i]);
        if (c->stage_ev[i]) cudaEventDestroy(c->stage_ev[i]);
    }
    if (c->arena) cudaFreeHost(c->arena);
    for (auto& s : c->spans) { cudaEventDestroy(s.a); cudaEventDestroy(s.b); }
    for (auto e : c->ev_pool) cudaEventDestroy(e);
    for (auto e : c->ev_chunks) cudaEventDestroy(e);
    cudaEventDestroy(c->ev_main);
    cudaStreamSynchronize(c->copy_stream);
    cudaStreamDestroy(c->copy_stream);
    cudaStreamDestroy(c->own_stream);
    delete c;
}

const char* hl_b200_label(hl_ctx* c) { return c ? c->label.c_str() : "hl_b200: no context"; }
const char* hl_b200_last_error(hl_ctx* c) {
    if (!c) return "no context";
    // a copy per calling thread: the text stays valid until this thread asks again, whatever the other threads decline meanwhile
    thread_local std::string mine;
    std::lock_guard<std::mutex> g(c->err_mu);
    mine = c->last_error;
    return mine.c_str();
}

int hl_b200_set_stream(hl_ctx* c, void* s) {
    if (!c) return HL_B200_ERR_ARG;
    std::lock_guard<std::mutex> g(c->mu);
    cudaStreamSynchronize(c->stream);
    c->stream = s ? (cudaStream_t)s : c->own_stream;
    return HL_B200_OK;
}

int hl_b200_sync(hl_ctx* c) {
    if (!c) return HL_B200_ERR_ARG;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    return sync(c, "synchronize");
}

int hl_b200_set_alloc_cap(hl_ctx* c, size_t bytes) {
    if (!c) return HL_B200_ERR_ARG;
    std::lock_guard<std::mutex> g(c->mu);
    c->alloc_cap = bytes;
    return HL_B200_OK;
}

int hl_b200_set_encoder(hl_ctx* c, int fast) {
    if (!c) return HL_B200_ERR_ARG;
    c->fast_encoder = fast != 0;
    return HL_B200_OK;
}

int hl_b200_set_slot_kernels(hl_ctx* c, int on) {
    if (!c) return HL_B200_ERR_ARG;
    c->slot_kernels = on != 0;
    return HL_B200_OK;
}

int hl_b200_stats(hl_ctx* c, hl_stats* out) {
    if (!c || !out) return HL_B200_ERR_ARG;
    std::lock_guard<std::mutex> g(c->mu);
    std::lock_guard<std::mutex> ge(c->err_mu);
    *out = c->stats;
    return HL_B200_OK;
}

int hl_b200_probe_field(hl_ctx* c, const uint64_t* a, const uint64_t* b, size_t n, uint64_t* out3n) {
    if (!c || (n && (!a || !b || !out3n))) return fail(c, HL_B200_ERR_ARG, "probe_field: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    u64 *da = nullptr, *db = nullptr, *dout = nullptr;
    int rc = dev_alloc(c, (void**)&da, n * 8);
    if (!rc) rc = dev_alloc(c, (void**)&db, n * 8);
    if (!rc) rc = dev_alloc(c, (void**)&dout, n * 24);
    if (!rc) rc = h2d(c, da, a, n * 8);
    if (!rc) rc = h2d(c, db, b, n * 8);
    if (!rc) {
        cudaError_t e = hlk::probe_field(da, db, n, dout, c->stream);
        c->stats.kernel_launches += n ? 1 : 0;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "probe_field launch", e);
    }
    if (!rc) rc = d2h(c, out3n, dout, n * 24);
    if (!rc) rc = sync(c, "probe_field");
    dev_free(c, da, n * 8); dev_free(c, db, n * 8); dev_free(c, dout, n * 24);
    return rc;
}

int hl_b200_butterfly_peak(hl_ctx* c, uint32_t iters, double* butterflies_per_second) {
    if (!c || !butterflies_per_second || iters == 0) return fail(c, HL_B200_ERR_ARG, "butterfly_peak: argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    std::vector<u64> seed(4096);
    u64 x = 88172645463325252ULL;
    for (auto& v : seed) { x ^= x << 13; x ^= x >> 7; x ^= x << 17; v = gl_canon(x); }
    u64 *d_seed = nullptr, *d_sink = nullptr;
    int rc = dev_alloc(c, (void**)&d_seed, 4096 * 8);
    if (!rc) rc = dev_alloc(c, (void**)&d_sink, 8);
    if (!rc) rc = h2d(c, d_seed, seed.data(), 4096 * 8);
    cudaEvent_t a = nullptr, b = nullptr;
    float ms = 0.f;
    const int blocks = c->sm_count * 8;
    if (!rc) {
        cudaEventCreate(&a); cudaEventCreate(&b);
        cudaError_t e = hlk::butterfly_peak(d_seed, d_sink, 8, blocks, c->stream);  // warm-up
        cudaEventRecord(a, c->stream);
        if (e == cudaSuccess) e = hlk::butterfly_peak(d_seed, d_sink, iters, blocks, c->stream);
        cudaEventRecord(b, c->stream);
        c->stats.kernel_launches += 2;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "butterfly_peak launch", e);
    }
    if (!rc) rc = sync(c, "butterfly_peak");
    if (!rc && cudaEventElapsedTime(&ms, a, b) != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "butterfly_peak timing");
    if (a) cudaEventDestroy(a);
    if (b) cudaEventDestroy(b);
    dev_free(c, d_seed, 4096 * 8); dev_free(c, d_sink, 8);
    if (!rc) *butterflies_per_second = (double)blocks * 256.0 * 32.0 * iters / (ms * 1e-3);
    return rc;
}

int hl_b200_compress_peak(hl_ctx* c, uint32_t iters, double* compressions_per_second) {
    if (!c || !compressions_per_second || iters == 0) return fail(c, HL_B200_ERR_ARG, "compress_peak: argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    std::vector<u64> seed(4096);
    u64 x = 88172645463325252ULL;
    for (auto& v : seed) { x ^= x << 13; x ^= x >> 7; x ^= x << 17; v = gl_canon(x); }
    u64 *d_seed = nullptr, *d_sink = nullptr;
    int rc = dev_alloc(c, (void**)&d_seed, 4096 * 8);
    if (!rc) rc = dev_alloc(c, (void**)&d_sink, 8);
    if (!rc) rc = h2d(c, d_seed, seed.data(), 4096 * 8);
    cudaEvent_t a = nullptr, b = nullptr;
    float ms = 0.f;
    const int blocks = c->sm_count * 16;
    if (!rc) {
        cudaEventCreate(&a); cudaEventCreate(&b);
        cudaError_t e = hlk::compress_peak(d_seed, d_sink, 8, blocks, c->stream);  // warm-up
        cudaEventRecord(a, c->stream);
        if (e == cudaSuccess) e = hlk::compress_peak(d_seed, d_sink, iters, blocks, c->stream);
        cudaEventRecord(b, c->stream);
        c->stats.kernel_launches += 2;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "compress_peak launch", e);
    }
    if (!rc) rc = sync(c, "compress_peak");
    if (!rc && cudaEventElapsedTime(&ms, a, b) != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "compress_peak timing");
    if (a) cudaEventDestroy(a);
    if (b) cudaEventDestroy(b);
    dev_free(c, d_seed, 4096 * 8); dev_free(c, d_sink, 8);
    if (!rc) *compressions_per_second = (double)blocks * 128.0 * iters / (ms * 1e-3);
    return rc;
}

}  // extern "C"
