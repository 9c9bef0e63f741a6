// C ABI: commitments (Backend::try_commit*), stores (EncodedStore), Merkle trees.
#include <cstring>
#include <thread>

#include "api_internal.h"

using namespace hlapi;

static int merkle_on_device(hl_ctx* c, const uint32_t* d_leaves, const uint32_t* d_salts, size_t nn, const uint8_t* leaf_key32,
                            const uint8_t* node_key32, uint32_t* d_levels) {
    uint32_t *d_lk = nullptr, *d_nk = nullptr;
    int rc = upload_key(c, leaf_key32, &d_lk);
    if (!rc) rc = upload_key(c, node_key32, &d_nk);
    if (!rc) {
        Timed t(c, HL_T_MERKLE);
        int launches = 0;
        const cudaError_t e = hlk::merkle_tree(d_leaves, d_salts, (u32)nn, d_lk, d_nk, d_levels, c->stream, &launches);
        c->stats.kernel_launches += launches;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "merkle launch", e);
    }
    if (d_lk) dev_free(c, d_lk, 32);
    if (d_nk) dev_free(c, d_nk, 32);
    return rc;
}

namespace {

struct Shape {
    u32 logn, logr, rows, q;
    bool zk;
};

// Where the data rows come from: NULL base = already in st->d_data; otherwise host memory, either 64-bit words (row_w NULL) or
// packed rows of 1-, 2-, 4- or 8-byte two's-complement words (row r at byte off[r], width row_w[r]).
struct HostRows {
    const void* base = nullptr;
    const uint8_t* row_w = nullptr;
    std::vector<u64> off;  // packed form only: rows + 1 byte offsets
    // what else the call brings from the host.  When the rows go up in pieces these ride with them instead of ahead of them: the
    // pads of a piece's rows behind the piece (st->d_pads is their place), `tail` (the salts: nothing reads them before the
    // tree) behind the last piece.  Otherwise both are copied before the rows.
    const u64* pads = nullptr;
    const void* tail_src = nullptr;
    void* tail_dst = nullptr;
    size_t tail_bytes = 0;
};

// Encode + column-hash.  With no host rows the data rows are already in st->d_data; otherwise they are
// uploaded here in row chunks on the context's copy stream while the encoder works on the chunks that
// have arrived (the upload of a block-sized matrix takes longer than its encoding).  Packed rows travel as
// their narrow bytes and are widened into st->d_data by the encoder's first pass.  Leaves stay in st->d_leaves.
int commit_on_device(hl_ctx* c, hl_store* st, const u64* d_pows, const uint8_t* key32, const HostRows& hr) {
    const u32 logn = st->logn, lognn = st->logn + st->logr;
    const size_t n = st->n(), nn = st->nn();
    // rows above 2^14 words run as 2 or 4 shared-memory transforms of 2^14 (encode_core.cuh)
    const u32 logb = logn > 14 ? 14u : logn, loga = logn - logb;
    const size_t nb = (size_t)1 << logb;
    const u32 T = st->zk ? (u32)((n + st->q + nb - 1) / nb) : (u32)(n / nb);
    const u64* tw = nullptr;
    int rc = root_powers(c, lognn, &tw);
    if (rc) return rc;
    const void* h_data = hr.base;
    const bool packed = h_data && hr.row_w;
    const bool fused_widen = packed && loga == 0 && logb >= 8 && c->fast_encoder;  // else a widening pass of its own per piece
    uint32_t* d_key = nullptr;
    u64* scratch = nullptr;
    uint32_t* cvs = nullptr;
    unsigned char *d_narrow = nullptr, *d_row_w = nullptr;
    u64* d_row_off = nullptr;
    const size_t scratch_words = hlk::encode_scratch_words(logb, T, c->sm_count, st->rows);
    const u32 nchunks = hlk::hash_chunks(st->rows);
    const size_t cvs_bytes = nchunks > 1 ? (size_t)nchunks * nn * 32 : 0;
    const size_t total_bytes = packed ? (size_t)hr.off[st->rows] : (size_t)st->rows * n * 8;
    rc = upload_key(c, key32, &d_key);
    if (!rc) rc = dev_alloc(c, (void**)&scratch, scratch_words * 8);
    if (!rc && cvs_bytes) rc = dev_alloc(c, (void**)&cvs, cvs_bytes);
    if (!rc && packed) rc = dev_alloc(c, (void**)&d_narrow, total_bytes + 16);
    if (!rc && packed) rc = dev_alloc(c, (void**)&d_row_off, (size_t)st->rows * 8);
    if (!rc && packed) rc = dev_alloc(c, (void**)&d_row_w, st->rows);
    if (!rc && packed) rc = h2d_owned(c, d_row_off, hr.off.data(), (size_t)st->rows * 8);
    if (!rc && packed) rc = h2d_owned(c, d_row_w, hr.row_w, st->rows);
    // Row pieces: a piece is encoded and its complete 1 KiB hash chunks (128 rows) are hashed while the next piece is still on
    // the bus.  Piece sizes are whole waves of the encoder (one row per SM per wave).  When the bytes per row make the bus the
    // slower side (64-bit words) the pieces are two waves and the last one a single wave, so that little follows the upload.
    // With narrow rows the device is the slower side when a GPU has the host's bus to itself, and the bus is the slower side again
    // when eight ranks upload at once (measured: the same 90 MB take 1.6 ms alone and 2.5-3.7 ms beside seven other ranks).  The
    // pieces are made for both: 1, 2, 3, 3, .. waves - the encoder starts after one wave's bytes, and no piece is more than 1.7
    // times its predecessor but the second, which is what keeps every next piece on the device before the encoder has finished the
    // one before it when the device is the slower side - and the last two waves as pieces of their own, so that one wave's
    // encoding, not five, follows the last byte when the bus is the slower side.
    auto byte_at = [&](u32 r) { return packed ? (size_t)hr.off[r] : (size_t)r * n * 8; };
    const u32 wave = (u32)c->sm_count;
    const bool split = h_data && total_bytes >= ((size_t)32 << 20) && st->rows > 4u * wave;
    const bool bus_bound = total_bytes / st->rows >= n * 6;  // bytes per row near the 64-bit form
    const bool pieces = split;
    std::vector<u32> piece_rows;
    if (!pieces) {
        piece_rows.push_back(st->rows);
    } else if (bus_bound) {
        for (u32 r0 = 0; r0 < st->rows;) {
            u32 nr = st->rows - r0 < 2u * wave ? st->rows - r0 : 2u * wave;
            if (r0 + nr == st->rows && nr > wave) nr -= wave;  // leave one wave or less for the end
            piece_rows.push_back(nr);
            r0 += nr;
        }
    } else {
        u32 rem = (st->rows + wave - 1) / wave, r0 = 0;  // waves left, the last one possibly short
        auto take = [&](u32 w) {
            const u32 nr = st->rows - r0 < w * wave ? st->rows - r0 : w * wave;
            piece_rows.push_back(nr);
            r0 += nr;
            rem -= w;
        };
        for (u32 w = 1; w <= 2 && rem > 2; w++) take(w < rem - 2 ? w : rem - 2);
        while (rem > 2) take(rem - 2 < 3 ? rem - 2 : 3);
        while (rem > 0) take(1);
    }
    if (!rc && pieces) {
        // the copy stream may touch the fresh allocations only after the main stream has made them
        cudaError_t e = cudaEventRecord(c->ev_main, c->stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(c->copy_stream, c->ev_main, 0);
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "stream ordering", e);
    }
    // Rows in ordinary pageable memory: the driver would stage them through its own buffer at about 10 GB/s, so the pieces go
    // through two page-locked buffers of the context instead, filled by a few host threads while the previous piece is on the bus.
    bool staged = false;
    if (!rc && pieces) {
        cudaPointerAttributes attr;
        const bool pageable = cudaPointerGetAttributes(&attr, h_data) != cudaSuccess || attr.type == cudaMemoryTypeUnregistered;
        cudaGetLastError();  // an unregistered pointer is not an error here
        size_t need = 0;  // the largest piece
        for (u32 r0 = 0, k = 0; k < piece_rows.size(); r0 += piece_rows[k++]) {
            const size_t b = byte_at(r0 + piece_rows[k]) - byte_at(r0);
            need = b > need ? b : need;
        }
        if (pageable) {
            staged = true;
            if (c->stage_bytes < need) {
                for (int i = 0; i < 2; i++) {
                    if (c->stage[i]) { cudaFreeHost(c->stage[i]); c->stage[i] = nullptr; }
                    if (cudaHostAlloc(&c->stage[i], need, cudaHostAllocDefault) != cudaSuccess) { c->stage[i] = nullptr; staged = false; }
                    if (!c->stage_ev[i] && cudaEventCreateWithFlags(&c->stage_ev[i], cudaEventDisableTiming) != cudaSuccess) staged = false;
                }
                c->stage_bytes = staged ? need : 0;
                cudaGetLastError();
            }
        }
    }
    if (!rc && !pieces && hr.pads) rc = h2d(c, st->d_pads, hr.pads, (size_t)st->rows * st->q * 8);
    if (!rc && !pieces && hr.tail_bytes) rc = h2d(c, hr.tail_dst, hr.tail_src, hr.tail_bytes);
    size_t piece_i = 0;
    if (!rc) {
        Timed t(c, HL_T_ENCODE);
        size_t ev_i = 0;
        u32 nr = 0, chunks_done = 0;
        size_t pk = 0;
        for (u32 r0 = 0; r0 < st->rows && !rc; r0 += nr) {
            nr = piece_rows[pk++];
            if (h_data) {
                cudaStream_t cs = pieces ? c->copy_stream : c->stream;
                const size_t b0 = byte_at(r0), bytes = byte_at(r0 + nr) - b0;
                const void* from = (const char*)h_data + b0;
                if (staged) {
                    const int b = (int)(piece_i++ & 1);
                    if (piece_i > 2) cudaEventSynchronize(c->stage_ev[b]);  // the copy that last read this buffer is done
                    const unsigned hw = std::thread::hardware_concurrency();
                    const int nth = bytes >= ((size_t)8 << 20) ? (int)(hw >= 8 ? 8 : hw >= 2 ? hw : 1) : 1;
                    std::vector<std::thread> th;
                    for (int k = 1; k < nth; k++)
                        th.emplace_back([=] { memcpy((char*)c->stage[b] + bytes * k / nth, (const char*)from + bytes * k / nth, bytes * (k + 1) / nth - bytes * k / nth); });
                    memcpy(c->stage[b], from, bytes / nth);
                    for (auto& x : th) x.join();
                    from = c->stage[b];
                }
                void* to = packed ? (void*)(d_narrow + b0) : (void*)(st->d_data + (size_t)r0 * n);
                cudaError_t e = cudaMemcpyAsync(to, from, bytes, cudaMemcpyHostToDevice, cs);
                if (staged && e == cudaSuccess) e = cudaEventRecord(c->stage_ev[(piece_i - 1) & 1], cs);
                c->stats.bytes_h2d += bytes;
                if (pieces && hr.pads && e == cudaSuccess) {
                    const size_t pb = (size_t)nr * st->q * 8;
                    e = cudaMemcpyAsync(st->d_pads + (size_t)r0 * st->q, hr.pads + (size_t)r0 * st->q, pb, cudaMemcpyHostToDevice, cs);
                    c->stats.bytes_h2d += pb;
                }
                if (pieces && hr.tail_bytes && r0 + nr == st->rows && e == cudaSuccess) {
                    e = cudaMemcpyAsync(hr.tail_dst, hr.tail_src, hr.tail_bytes, cudaMemcpyHostToDevice, cs);
                    c->stats.bytes_h2d += hr.tail_bytes;
                }
                if (e == cudaSuccess && cs != c->stream) {
                    if (ev_i == c->ev_chunks.size()) {
                        cudaEvent_t ev = nullptr;
                        e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
                        if (e == cudaSuccess) c->ev_chunks.push_back(ev);
                    }
                    if (e == cudaSuccess) e = cudaEventRecord(c->ev_chunks[ev_i], cs);
                    if (e == cudaSuccess) e = cudaStreamWaitEvent(c->stream, c->ev_chunks[ev_i], 0);
                    ev_i++;
                }
                if (e != cudaSuccess) { rc = fail(c, HL_B200_ERR_DEVICE, "row upload", e); break; }
            }
            if (packed && !fused_widen) {
                cudaError_t e = hlk::widen_rows(d_narrow, d_row_off + r0, d_row_w + r0, st->d_data + (size_t)r0 * n, nr, (u32)n, c->sm_count, c->stream);
                c->stats.kernel_launches += 1;
                if (e != cudaSuccess) { rc = fail(c, HL_B200_ERR_DEVICE, "row widening launch", e); break; }
            }
            enc::RowArgs a;
            a.data = st->d_data + (size_t)r0 * n;
            a.pads = st->d_pads ? st->d_pads + (size_t)r0 * st->q : nullptr;
            a.pows = d_pows; a.tw_nn = tw; a.enc = st->d_enc + (size_t)r0 * nn; a.scratch = scratch;
            a.rows = nr; a.q = st->zk ? st->q : 0; a.T = T; a.logr = st->logr + loga; a.loga = loga; a.zk = st->zk ? 1 : 0;
            a.ninv = gl_inv((u64)n); a.coef_out = nullptr;
            if (fused_widen) { a.narrow = d_narrow; a.row_off = d_row_off + r0; a.row_w = d_row_w + r0; }
            // a handful of rows (a boundary commitment, the last piece of an upload): one CTA per (row, residue)
            a.split = (loga == 0 && st->logr >= 1 && ((u64)nr << st->logr) <= (u64)c->sm_count) ? 1 : 0;
            cudaError_t e = hlk::encode_rows(a, logb, c->fast_encoder || loga, c->sm_count, scratch_words, c->stream, &st->encoder_path);
            c->stats.kernel_launches += 1;
            if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "row encoder launch", e);
            // the 128-row hash chunks that are complete now.  Launches of one or two chunks fill the machine badly (five such
            // launches took 430 us against 350 us for all twenty chunks in one), so narrow rows wait until four chunks are
            // ready; the last launch takes what is left.
            if (!rc && pieces) {
                const u32 c1 = r0 + nr == st->rows ? nchunks : (r0 + nr) / 128u;
                if (c1 > chunks_done && (bus_bound || c1 - chunks_done >= 4 || r0 + nr == st->rows)) {
                    e = hlk::hash_column_chunks(st->d_enc, st->rows, (u32)nn, d_key, chunks_done, c1 - chunks_done, cvs, st->d_leaves, c->stream);
                    c->stats.kernel_launches += 1;
                    if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "column hash launch", e);
                    chunks_done = c1;
                }
            }
        }
    }
    if (!rc && pieces) {
        Timed t(c, HL_T_HASH);
        cudaError_t e = hlk::hash_column_merge(st->rows, (u32)nn, d_key, cvs, st->d_leaves, c->stream);
        c->stats.kernel_launches += 1;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "column hash merge launch", e);
    }
    if (!rc && !pieces) {
        Timed t(c, HL_T_HASH);
        cudaError_t e = hlk::hash_columns(st->d_enc, st->rows, (u32)nn, d_key, cvs, st->d_leaves, c->stream);
        c->stats.kernel_launches += nchunks > 1 ? 2 : 1;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "column hash launch", e);
    }
    dev_free(c, scratch, scratch_words * 8);
    if (cvs) dev_free(c, cvs, cvs_bytes);
    if (d_key) dev_free(c, d_key, 32);
    if (d_narrow) dev_free(c, d_narrow, total_bytes + 16);
    if (d_row_off) dev_free(c, d_row_off, (size_t)st->rows * 8);
    if (d_row_w) dev_free(c, d_row_w, st->rows);
    return rc;
}

int check_shape(hl_ctx* c, uint32_t log_cols, uint32_t inv_rate, size_t rows, size_t q, bool zk, uint32_t max_log, Shape* s) {
    int logr = log2_exact(inv_rate);
    if (logr < 0 || rows == 0 || rows > 0x7FFFFFFFu) return fail(c, HL_B200_ERR_ARG, "commit: rows or inv_rate");
    if (log_cols < 1) return fail(c, HL_B200_ERR_UNSUPPORTED, "commit: fewer than 2 columns");
    if (log_cols > 16) return fail(c, HL_B200_ERR_UNSUPPORTED, "commit: more than 2^16 columns per row");
    if (max_log && log_cols + (uint32_t)logr > max_log) return fail(c, HL_B200_ERR_ARG, "commit: transform exceeds the caller's NTT tables");
    size_t n = (size_t)1 << log_cols, nn = n << logr;
    if (zk && (q == 0 || n + q > nn)) return fail(c, HL_B200_ERR_ARG, "commit_zk: pad count (need 0 < q and n + q <= nn)");
    if (rows * nn > ((size_t)1 << 36)) return fail(c, HL_B200_ERR_UNSUPPORTED, "commit: encoding above 512 GiB");
    s->logn = log_cols; s->logr = (u32)logr; s->rows = (u32)rows; s->q = zk ? (u32)q : 0; s->zk = zk;
    return HL_B200_OK;
}

void free_store(hl_store* st) {
    hl_ctx* c = st->ctx;
    c->stores.erase(st);
    if (st->owns_inputs) {
        dev_free(c, st->d_data, (size_t)st->rows * st->n() * 8);
        dev_free(c, st->d_pads, (size_t)st->rows * st->q * 8);
    }
    dev_free(c, st->d_enc, (size_t)st->rows * st->nn() * 8);
    dev_free(c, st->d_leaves, st->nn() * 32);
    delete st;
}

// the salted tree to build in the same call (commit_zk_owned_with_tag draws the salts before it offers the commitment, pcs.rs:788-792)
struct TreeAsk {
    const uint8_t *salts32, *leaf_key32, *node_key32;
    uint8_t* levels_out;
};

int commit_host(hl_ctx* c, const Shape& s, const HostRows& data, const uint64_t* pads, const uint64_t* pows,
                const uint8_t* key32, hl_store** store, uint8_t* leaves32, const TreeAsk* tree = nullptr) {
    hl_store* st = new hl_store();
    st->ctx = c; st->rows = s.rows; st->logn = s.logn; st->logr = s.logr; st->q = s.q; st->zk = s.zk;
    const size_t n = st->n(), nn = st->nn();
    u64* d_pows = nullptr;
    uint32_t *d_salts = nullptr, *d_levels = nullptr;
    int rc = dev_alloc(c, (void**)&st->d_data, (size_t)s.rows * n * 8);
    if (!rc && tree) rc = dev_alloc(c, (void**)&d_salts, nn * 32);
    if (!rc && tree) rc = dev_alloc(c, (void**)&d_levels, (2 * nn - 1) * 32);
    if (!rc && s.zk) rc = dev_alloc(c, (void**)&st->d_pads, (size_t)s.rows * s.q * 8);
    if (!rc && s.zk) rc = dev_alloc(c, (void**)&d_pows, nn * 8);
    if (!rc) rc = dev_alloc(c, (void**)&st->d_enc, (size_t)s.rows * nn * 8);
    if (!rc) rc = dev_alloc(c, (void**)&st->d_leaves, nn * 32);
    if (!rc && s.zk) rc = h2d(c, d_pows, pows, nn * 8);
    HostRows hr = data;  // the pads and the salts travel with the rows (commit_on_device)
    if (s.zk) hr.pads = reinterpret_cast<const u64*>(pads);
    if (tree) { hr.tail_src = tree->salts32; hr.tail_dst = d_salts; hr.tail_bytes = nn * 32; }
    if (!rc) rc = commit_on_device(c, st, d_pows, key32, hr);
    if (!rc && tree) rc = merkle_on_device(c, st->d_leaves, d_salts, nn, tree->leaf_key32, tree->node_key32, d_levels);
    if (!rc && leaves32) rc = d2h(c, leaves32, st->d_leaves, nn * 32);
    if (!rc && tree) rc = d2h(c, tree->levels_out, d_levels, (2 * nn - 1) * 32);
    if (!rc) rc = sync(c, "commit");
    if (!rc && tree) c->stats.merkles++;
    if (d_pows) dev_free(c, d_pows, nn * 8);
    if (d_salts) dev_free(c, d_salts, nn * 32);
    if (d_levels) dev_free(c, d_levels, (2 * nn - 1) * 32);
    if (rc) { cudaStreamSynchronize(c->copy_stream); cudaStreamSynchronize(c->stream); free_store(st); return rc; }
    c->stats.commits++;
    c->stores.insert(st);
    *store = st;
    return HL_B200_OK;
}

}  // namespace

void hlapi::store_release(hl_store* st) { free_store(st); }

// hl_b200_commit_zk_dev without the lock: for entry points that hold it already
int hlapi::commit_resident(hl_ctx* c, u32 log_cols, u32 inv_rate, const u64* d_data, size_t rows, const u64* d_pads, size_t q, const u64* d_pows,
                           const uint8_t* key32, hl_store** store, uint8_t* d_leaves32) {
    Shape s;
    int rc = check_shape(c, log_cols, inv_rate, rows, q, true, 0, &s);
    if (rc) return rc;
    hl_store* st = new hl_store();
    st->ctx = c; st->rows = s.rows; st->logn = s.logn; st->logr = s.logr; st->q = s.q; st->zk = true;
    st->owns_inputs = false;
    st->d_data = const_cast<u64*>(d_data);
    st->d_pads = const_cast<u64*>(d_pads);
    const size_t nn = st->nn();
    rc = dev_alloc(c, (void**)&st->d_enc, (size_t)s.rows * nn * 8);
    if (!rc) rc = dev_alloc(c, (void**)&st->d_leaves, nn * 32);
    if (!rc) rc = commit_on_device(c, st, d_pows, key32, HostRows());
    if (!rc && d_leaves32) {
        cudaError_t e = cudaMemcpyAsync(d_leaves32, st->d_leaves, nn * 32, cudaMemcpyDeviceToDevice, c->stream);
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "leaf copy", e);
    }
    if (rc) { cudaStreamSynchronize(c->stream); free_store(st); return rc; }
    c->stats.commits++;
    c->stores.insert(st);
    *store = st;
    return HL_B200_OK;
}

extern "C" {

int hl_b200_commit(hl_ctx* c, uint32_t log_cols, uint32_t inv_rate, const uint64_t* data, size_t rows, uint32_t max_log,
                   const uint8_t* key32, hl_store** store, uint8_t* leaves32) {
    if (!c || !data || !store || !leaves32) return fail(c, HL_B200_ERR_ARG, "commit: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    Shape s;
    int rc = check_shape(c, log_cols, inv_rate, rows, 0, false, max_log, &s);
    if (rc) return rc;
    HostRows hr;
    hr.base = data;
    return commit_host(c, s, hr, nullptr, nullptr, key32, store, leaves32);
}

int hl_b200_commit_zk(hl_ctx* c, uint32_t log_cols, uint32_t inv_rate, const uint64_t* data, size_t rows,
                      const uint64_t* pads, size_t q, const uint64_t* pows, uint32_t max_log, const uint8_t* key32,
                      hl_store** store, uint8_t* leaves32) {
    if (!c || !data || !pads || !pows || !store || !leaves32) return fail(c, HL_B200_ERR_ARG, "commit_zk: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    Shape s;
    int rc = check_shape(c, log_cols, inv_rate, rows, q, true, max_log, &s);
    if (rc) return rc;
    HostRows hr;
    hr.base = data;
    return commit_host(c, s, hr, pads, pows, key32, store, leaves32);
}

int hl_b200_commit_zk_tree(hl_ctx* c, uint32_t log_cols, uint32_t inv_rate, const uint64_t* data, size_t rows, const uint64_t* pads, size_t q,
                           const uint64_t* pows, uint32_t max_log, const uint8_t* key32, const uint8_t* salts32, const uint8_t* leaf_key32,
                           const uint8_t* node_key32, hl_store** store, uint8_t* leaves32, uint8_t* levels_out) {
    if (!c || !data || !pads || !pows || !salts32 || !store || !levels_out) return fail(c, HL_B200_ERR_ARG, "commit_zk_tree: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    Shape s;
    int rc = check_shape(c, log_cols, inv_rate, rows, q, true, max_log, &s);
    if (rc) return rc;
    const TreeAsk tree{salts32, leaf_key32, node_key32, levels_out};
    HostRows hr;
    hr.base = data;
    return commit_host(c, s, hr, pads, pows, key32, store, leaves32, &tree);
}

int hl_b200_commit_zk_packed(hl_ctx* c, uint32_t log_cols, uint32_t inv_rate, const void* packed, const uint8_t* row_width, size_t rows,
                             const uint64_t* pads, size_t q, const uint64_t* pows, uint32_t max_log, const uint8_t* key32, const uint8_t* salts32,
                             const uint8_t* leaf_key32, const uint8_t* node_key32, hl_store** store, uint8_t* leaves32, uint8_t* levels_out) {
    if (!c || !packed || !row_width || !pads || !pows || !store || (salts32 && !levels_out) || (!salts32 && !leaves32))
        return fail(c, HL_B200_ERR_ARG, "commit_zk_packed: null argument");
    Shape s;
    HostRows hr;
    if (int rc = check_shape(c, log_cols, inv_rate, rows, q, true, max_log, &s)) return rc;
    if (log_cols < 3) return fail(c, HL_B200_ERR_UNSUPPORTED, "commit_zk_packed: rows of fewer than 8 words");  // keeps every row 8-byte aligned
    hr.base = packed;
    hr.row_w = row_width;
    hr.off.resize(rows + 1);
    u64 at = 0;
    for (size_t r = 0; r < rows; r++) {
        const uint8_t w = row_width[r];
        if (w != 1 && w != 2 && w != 4 && w != 8) return fail(c, HL_B200_ERR_ARG, "commit_zk_packed: a row width other than 1, 2, 4 or 8 bytes");
        hr.off[r] = at;
        at += (u64)w << log_cols;
    }
    hr.off[rows] = at;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    if (salts32) {
        const TreeAsk tree{salts32, leaf_key32, node_key32, levels_out};
        return commit_host(c, s, hr, pads, pows, key32, store, leaves32, &tree);
    }
    return commit_host(c, s, hr, pads, pows, key32, store, leaves32);
}

int hl_b200_commit_zk_dev(hl_ctx* c, uint32_t log_cols, uint32_t inv_rate, const uint64_t* d_data, size_t rows,
                          const uint64_t* d_pads, size_t q, const uint64_t* d_pows, const uint8_t* key32,
                          hl_store** store, uint8_t* d_leaves32) {
    if (!c || !d_data || !d_pads || !d_pows || !store) return fail(c, HL_B200_ERR_ARG, "commit_zk_dev: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    return commit_resident(c, log_cols, inv_rate, (const u64*)d_data, rows, (const u64*)d_pads, q, (const u64*)d_pows, key32, store, d_leaves32);
}

int hl_b200_store_shape(hl_store* st, size_t* rows, size_t* n, size_t* nn, size_t* q) {
    if (!st) return HL_B200_ERR_ARG;
    if (rows) *rows = st->rows;
    if (n) *n = st->n();
    if (nn) *nn = st->nn();
    if (q) *q = st->q;
    return HL_B200_OK;
}

const uint64_t* hl_b200_store_encoded_dev(hl_store* st) { return st ? (const uint64_t*)st->d_enc : nullptr; }
const uint8_t* hl_b200_store_leaves_dev(hl_store* st) { return st ? (const uint8_t*)st->d_leaves : nullptr; }

void hl_b200_store_free(hl_store* st) {
    if (!st) return;
    hl_ctx* c = st->ctx;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    free_store(st);
}

int hl_b200_store_fold(hl_store* st, const uint64_t* rhos, size_t k, int with_pads, uint64_t* out) {
    if (!st) return HL_B200_ERR_ARG;
    hl_ctx* c = st->ctx;
    if (k && (!rhos || !out)) return fail(c, HL_B200_ERR_ARG, "store_fold: null argument");
    if (with_pads && !st->zk) return fail(c, HL_B200_ERR_ARG, "store_fold: pads asked of a plain store");
    if (k == 0) return HL_B200_OK;
    if (k > 0xFFFFu * 8u) return fail(c, HL_B200_ERR_ARG, "store_fold: too many vectors");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    const u32 n = (u32)st->n(), q = with_pads ? st->q : 0, w = n + q, rows = st->rows;
    // An opening's group vectors are zero outside their claims' rows (pcs.rs:851-891), its proximity vector is dense.
    // Vectors with few non-zero rows go to the list kernel, the others to the dense one; both write the caller's order.
    std::vector<u32> dense_map, sparse_map, s_off{0}, s_rows;
    std::vector<u64> dense_rhos, s_w;
    for (size_t g = 0; g < k; g++) {
        const uint64_t* r = rhos + g * (size_t)rows * 2;
        u32 support = 0;
        for (u32 i = 0; i < rows; i++) support += (r[2 * i] | r[2 * i + 1]) != 0;
        if (support * 8u <= rows) {
            for (u32 i = 0; i < rows; i++)
                if (r[2 * i] | r[2 * i + 1]) { s_rows.push_back(i); s_w.push_back(r[2 * i]); s_w.push_back(r[2 * i + 1]); }
            s_off.push_back((u32)s_rows.size());
            sparse_map.push_back((u32)g);
        } else {
            dense_rhos.insert(dense_rhos.end(), r, r + (size_t)rows * 2);
            dense_map.push_back((u32)g);
        }
    }
    const u32 kd = (u32)dense_map.size(), ks = (u32)sparse_map.size();
    u64 *d_rhos = nullptr, *d_out = nullptr, *d_sw = nullptr;
    u32 *d_dmap = nullptr, *d_smap = nullptr, *d_soff = nullptr, *d_srows = nullptr;
    const size_t rb = (size_t)(kd ? kd : 1) * rows * 16, ob = k * (size_t)w * 16, ne = s_rows.size() ? s_rows.size() : 1;
    int rc = dev_alloc(c, (void**)&d_out, ob);
    if (!rc && kd) {
        rc = dev_alloc(c, (void**)&d_rhos, rb);
        if (!rc) rc = dev_alloc(c, (void**)&d_dmap, kd * 4);
        if (!rc) rc = h2d(c, d_rhos, dense_rhos.data(), (size_t)kd * rows * 16);
        if (!rc) rc = h2d(c, d_dmap, dense_map.data(), kd * 4);
    }
    if (!rc && ks) {
        rc = dev_alloc(c, (void**)&d_smap, ks * 4);
        if (!rc) rc = dev_alloc(c, (void**)&d_soff, (ks + 1) * 4);
        if (!rc) rc = dev_alloc(c, (void**)&d_srows, ne * 4);
        if (!rc) rc = dev_alloc(c, (void**)&d_sw, ne * 16);
        if (!rc) rc = h2d(c, d_smap, sparse_map.data(), ks * 4);
        if (!rc) rc = h2d(c, d_soff, s_off.data(), (ks + 1) * 4);
        if (!rc && s_rows.size()) rc = h2d(c, d_srows, s_rows.data(), s_rows.size() * 4);
        if (!rc && s_rows.size()) rc = h2d(c, d_sw, s_w.data(), s_w.size() * 8);
    }
    const bool contiguous = st->zk || st->fold_data;
    const u32 few = kd ? hlk::fold_few_ranges(rows, n, q, kd, contiguous ? 1u : 2u, c->sm_count) : 0;
    const u32 fsplits = kd && !few ? hlk::fold_row_splits(rows, n, q, kd, c->sm_count) : 1;
    u64* d_part = nullptr;
    const size_t part_bytes = few ? (size_t)few * kd * w * 16 : fsplits > 1 ? (size_t)fsplits * kd * w * 16 : 0;
    if (!rc && part_bytes) rc = dev_alloc(c, (void**)&d_part, part_bytes);
    if (!rc) {
        Timed t(c, HL_T_FOLD);
        // hiding form: the message is the resident data (the encoding is not systematic, pcs.rs:985-987);
        // plain form: the systematic positions of the encoding (pcs.rs:332-340)
        const bool from_data = st->zk || st->fold_data;
        const u64* src = from_data ? st->d_data : st->d_enc;
        const size_t ld = from_data ? n : st->nn();
        const u32 ir = from_data ? 1u : 1u << st->logr;
        const u64* src2 = st->zk && q ? st->d_pads : nullptr;
        cudaError_t e = cudaSuccess;
        if (kd && few) {
            e = hlk::fold_rows_few(src, rows, n, ld, src2, q, q, d_rhos, kd, d_dmap, d_out, w, few, d_part, c->stream);
            c->stats.kernel_launches += 2;
        } else if (kd) {
            e = hlk::fold_rows(src, rows, n, ld, ir, src2, q, q, d_rhos, kd, d_dmap, d_out, w, c->stream, fsplits, d_part);
            c->stats.kernel_launches += fsplits > 1 ? 2 : 1;
        }
        if (e == cudaSuccess && ks) {
            e = hlk::fold_rows_sparse(src, n, ld, ir, src2, q, q, d_soff, d_srows, d_sw, ks, d_smap, d_out, w, c->stream);
            c->stats.kernel_launches++;
        }
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "fold launch", e);
    }
    if (!rc) rc = d2h(c, out, d_out, ob);
    if (!rc) rc = sync(c, "store_fold");
    if (d_part) dev_free(c, d_part, part_bytes);
    if (d_rhos) dev_free(c, d_rhos, rb);
    if (d_dmap) dev_free(c, d_dmap, kd * 4);
    if (d_smap) dev_free(c, d_smap, ks * 4);
    if (d_soff) dev_free(c, d_soff, (ks + 1) * 4);
    if (d_srows) dev_free(c, d_srows, ne * 4);
    if (d_sw) dev_free(c, d_sw, ne * 16);
    if (d_out) dev_free(c, d_out, ob);
    if (!rc) c->stats.folds++;
    return rc;
}

int hl_b200_store_columns(hl_store* st, const uint64_t* idx, size_t nidx, uint64_t* out) {
    if (!st) return HL_B200_ERR_ARG;
    hl_ctx* c = st->ctx;
    if (nidx && (!idx || !out)) return fail(c, HL_B200_ERR_ARG, "store_columns: null argument");
    if (nidx == 0) return HL_B200_OK;
    if (nidx > 65535) return fail(c, HL_B200_ERR_ARG, "store_columns: more than 65535 columns in one call");
    for (size_t i = 0; i < nidx; i++)
        if (idx[i] >= st->nn()) return fail(c, HL_B200_ERR_ARG, "store_columns: index out of range");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    u64 *d_idx = nullptr, *d_out = nullptr;
    const size_t ob = nidx * (size_t)st->rows * 8;
    int rc = dev_alloc(c, (void**)&d_idx, nidx * 8);
    if (!rc) rc = dev_alloc(c, (void**)&d_out, ob);
    if (!rc) rc = h2d(c, d_idx, idx, nidx * 8);
    if (!rc) {
        Timed t(c, HL_T_GATHER);
        cudaError_t e = hlk::gather_columns(st->d_enc, st->rows, st->nn(), d_idx, (u32)nidx, d_out, c->stream);
        c->stats.kernel_launches++;
        if (e != cudaSuccess) rc = fail(c, HL_B200_ERR_DEVICE, "gather launch", e);
    }
    if (!rc) rc = d2h(c, out, d_out, ob);
    if (!rc) rc = sync(c, "store_columns");
    dev_free(c, d_idx, nidx * 8); dev_free(c, d_out, ob);
    if (!rc) c->stats.gathers++;
    return rc;
}

// salted leaves + all levels into d_levels, from device leaves (and device salts, or none)
static int merkle_common(hl_ctx* c, const uint32_t* d_leaves_in, const uint8_t* h_leaves, const uint8_t* salts32, size_t nn,
                         const uint8_t* leaf_key32, const uint8_t* node_key32, uint8_t* levels_out) {
    if (log2_exact(nn) < 0 || nn > ((size_t)1 << 26)) return fail(c, HL_B200_ERR_ARG, "merkle: leaf count must be a power of two");
    const size_t lv_bytes = (2 * nn - 1) * 32;
    uint32_t *d_levels = nullptr, *d_in = nullptr, *d_salts = nullptr;
    int rc = dev_alloc(c, (void**)&d_levels, lv_bytes);
    const uint32_t* leaves = d_leaves_in;
    if (!rc && !leaves) {
        rc = dev_alloc(c, (void**)&d_in, nn * 32);
        if (!rc) rc = h2d(c, d_in, h_leaves, nn * 32);
        leaves = d_in;
    }
    if (!rc && salts32) {
        rc = dev_alloc(c, (void**)&d_salts, nn * 32);
        if (!rc) rc = h2d(c, d_salts, salts32, nn * 32);
    }
    if (!rc) rc = merkle_on_device(c, leaves, d_salts, nn, leaf_key32, node_key32, d_levels);
    if (!rc) rc = d2h(c, levels_out, d_levels, lv_bytes);
    if (!rc) rc = sync(c, "merkle");
    dev_free(c, d_levels, lv_bytes);
    if (d_in) dev_free(c, d_in, nn * 32);
    if (d_salts) dev_free(c, d_salts, nn * 32);
    if (!rc) c->stats.merkles++;
    return rc;
}

int hl_b200_merkle(hl_ctx* c, const uint8_t* leaves32, const uint8_t* salts32, size_t nn, const uint8_t* leaf_key32,
                   const uint8_t* node_key32, uint8_t* levels_out) {
    if (!c || !leaves32 || !levels_out) return fail(c, HL_B200_ERR_ARG, "merkle: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    return merkle_common(c, nullptr, leaves32, salts32, nn, leaf_key32, node_key32, levels_out);
}

int hl_b200_store_merkle(hl_store* st, const uint8_t* salts32, const uint8_t* leaf_key32, const uint8_t* node_key32,
                         uint8_t* levels_out) {
    if (!st || !levels_out) return HL_B200_ERR_ARG;
    hl_ctx* c = st->ctx;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    return merkle_common(c, st->d_leaves, nullptr, salts32, st->nn(), leaf_key32, node_key32, levels_out);
}

int hl_b200_store_merkle_dev(hl_store* st, const uint8_t* d_salts32, const uint8_t* leaf_key32, const uint8_t* node_key32,
                             uint8_t* d_levels_out) {
    if (!st || !d_levels_out) return HL_B200_ERR_ARG;
    hl_ctx* c = st->ctx;
    // the tree kernels move digests as 16-byte vectors: a misaligned caller pointer would be a device fault, not a status
    if (((uintptr_t)d_levels_out & 15) || ((uintptr_t)d_salts32 & 15)) return fail(c, HL_B200_ERR_ARG, "store_merkle_dev: device pointers must be 16-byte aligned");
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    int rc = merkle_on_device(c, st->d_leaves, (const uint32_t*)d_salts32, st->nn(), leaf_key32, node_key32, (uint32_t*)d_levels_out);
    if (!rc) c->stats.merkles++;
    return rc;
}

}  // extern "C"
