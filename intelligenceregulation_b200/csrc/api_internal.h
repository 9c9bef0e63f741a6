// Host-side objects behind the opaque handles of include/hl_b200.h.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <set>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/hl_b200.h"
#include "kernels.h"

struct hl_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;     // uploads that overlap the encoder
    cudaEvent_t ev_main = nullptr;
    std::vector<cudaEvent_t> ev_chunks;
    bool fast_encoder = true;
    bool slot_kernels = false;  // run a slot program whose graph is known through its generated kernel instead of the interpreter (measured slower: off)
    std::mutex mu;
    std::mutex err_mu;       // guards last_error and stats.declines: a decline may be recorded before `mu` is taken, from any thread
    std::map<u32, u64*> tw;  // log2 nn -> nn powers of the nn-th root
    std::string label, last_error;
    hl_stats stats{};
    bool timing = false;
    struct Span { cudaEvent_t a, b; int cls; };
    std::vector<Span> spans;          // recorded, not yet read
    std::vector<cudaEvent_t> ev_pool;  // events ready for reuse
    hl_timing timing_acc{};
    void* stage[2] = {nullptr, nullptr};       // page-locked staging for uploads from pageable host memory (lazily allocated)
    size_t stage_bytes = 0;
    cudaEvent_t stage_ev[2] = {nullptr, nullptr};  // the copy out of stage[i] has completed
    char* arena = nullptr;     // page-locked bounce area for small caller-owned inputs of calls that return before their copies run
    size_t arena_off = 0;
    int* d_wp_flag = nullptr;  // the witness products' status word: zero between calls
    bool wp_attr = false;      // the product kernel's shared-memory size has been raised on this device
    std::set<const struct hl_store*> stores;  // the live commitment stores (a planned slot table that reads one checks it is still there when it is built)
    size_t alloc_live = 0;   // bytes handed out and not yet returned
    size_t alloc_cap = 0;    // 0 = none; a host-side failure-injection cap (mod.rs:121 set_alloc_cap_for_test)
};

struct hl_store {
    hl_ctx* ctx = nullptr;
    u32 rows = 0, logn = 0, logr = 0, q = 0;
    bool zk = false;
    bool owns_inputs = true;      // false: d_data / d_pads belong to the caller
    bool fold_data = false;       // a plain store whose row fold reads d_data (a masking commitment's coefficient rows)
    u64* d_data = nullptr;        // rows x n
    u64* d_pads = nullptr;        // rows x q
    u64* d_enc = nullptr;         // rows x nn
    uint32_t* d_leaves = nullptr; // nn x 8 words, unsalted
    int encoder_path = -1;
    size_t n() const { return (size_t)1 << logn; }
    size_t nn() const { return (size_t)1 << (logn + logr); }
};

namespace hlapi {
int fail(hl_ctx* c, int code, const char* what, cudaError_t e = cudaSuccess);
int dev_alloc(hl_ctx* c, void** p, size_t bytes);
void dev_free(hl_ctx* c, void* p, size_t bytes);
int h2d(hl_ctx* c, void* d, const void* h, size_t bytes);
int d2h(hl_ctx* c, void* h, const void* d, size_t bytes);
// like h2d, but the caller's bytes are no longer needed when it returns, whatever kind of host memory they live in
int h2d_owned(hl_ctx* c, void* d, const void* h, size_t bytes);
int sync(hl_ctx* c, const char* what);
int root_powers(hl_ctx* c, u32 lognn, const u64** out);
int upload_key(hl_ctx* c, const uint8_t* key32, uint32_t** d_key);
int log2_exact(size_t v);
void store_release(hl_store* st);  // frees a store; the caller holds the context's lock
// a hiding commitment of rows that are on the device already (hl_b200_commit_zk_dev); the caller holds the context's lock
int commit_resident(hl_ctx* c, u32 log_cols, u32 inv_rate, const u64* d_data, size_t rows, const u64* d_pads, size_t q, const u64* d_pows,
                    const uint8_t* key32, hl_store** store, uint8_t* d_leaves32);

// Brackets the launches of one kernel family with two events when the context's timing is on.
struct Timed {
    hl_ctx* c;
    hl_ctx::Span s;
    bool on;
    Timed(hl_ctx* c, int cls);
    ~Timed();
};
}  // namespace hlapi
