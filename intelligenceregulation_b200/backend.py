"""Host-side mirror of the prover's accelerator seam over the C ABI.

The reference reaches a device through ``trait Backend`` / ``trait EncodedStore``
(zkp-core/src/pcs/backend.rs:30-100) and hashline's adapter
(hashline/src/gpu/mod.rs:687-859: ``backend()``, ``enabled()``, ``label()``, ``DevStore``).
The names, argument meaning and error behaviour here follow those: a hook returns
``None`` when the device declines (the error is counted and kept in ``declined``),
and raises instead when ``HL_GPU_REQUIRED=1`` (mod.rs:76-102).  Arrays are numpy
``uint64`` (canonical Goldilocks words; an Fp2 is two consecutive words).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Tuple

import numpy as np

from . import _lib


def _ptr(a) -> C.c_void_p:
    if a is None:
        return C.c_void_p(0)
    if isinstance(a, (bytes, bytearray)):
        return C.cast(C.create_string_buffer(bytes(a), len(a)), C.c_void_p)
    if isinstance(a, int):
        return C.c_void_p(a)
    assert a.flags["C_CONTIGUOUS"]
    return C.c_void_p(a.ctypes.data)


def _u64(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint64)


def required() -> bool:
    """hashline/src/gpu/mod.rs:76-78."""
    return os.environ.get("HL_GPU_REQUIRED") == "1"


class DeviceError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"hl_b200 error {code}: {text}")
        self.code = code


class Context:
    """One device context (hashline/src/gpu/metal.rs:75-95 keeps one per process)."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        h = C.c_void_p()
        rc = self.lib.hl_b200_init(device, C.byref(h))
        if rc != 0:
            raise DeviceError(rc, "no usable CUDA device")
        self.h = h
        self.declines: List[Tuple[str, str]] = []

    def close(self) -> None:
        if self.h:
            self.lib.hl_b200_shutdown(self.h)
            self.h = None

    def label(self) -> str:
        return self.lib.hl_b200_label(self.h).decode()

    def last_error(self) -> str:
        return self.lib.hl_b200_last_error(self.h).decode()

    def check(self, rc: int) -> None:
        if rc != 0:
            raise DeviceError(rc, self.last_error())

    def declined(self, site: str, rc: int) -> None:
        """mod.rs:80-94: log and count a decline; under HL_GPU_REQUIRED=1 a decline is fatal."""
        text = self.last_error()
        self.declines.append((site, text))
        if required():
            raise DeviceError(rc, f"{site}: {text} (HL_GPU_REQUIRED=1)")

    def set_stream(self, cuda_stream: int) -> None:
        self.check(self.lib.hl_b200_set_stream(self.h, C.c_void_p(cuda_stream)))

    def set_encoder(self, fast: bool) -> None:
        self.check(self.lib.hl_b200_set_encoder(self.h, 1 if fast else 0))

    def set_slot_kernels(self, on: bool) -> None:
        """the generated per-graph round kernels, or (default) the interpreter, for slot programs with a known graph"""
        self.check(self.lib.hl_b200_set_slot_kernels(self.h, 1 if on else 0))

    def set_dependent_launch(self, on: bool) -> None:
        """measurement aid (process-wide): the sumcheck kernels as a programmatic dependent-launch chain (default) or as ordinary launches"""
        self.check(self.lib.hl_b200_set_dependent_launch(1 if on else 0))

    def set_alloc_cap(self, nbytes: int) -> None:
        """Host-side allocation-failure injection (0 = no cap)."""
        self.check(self.lib.hl_b200_set_alloc_cap(self.h, nbytes))

    def sync(self) -> None:
        self.check(self.lib.hl_b200_sync(self.h))

    def stats(self) -> dict:
        s = _lib.Stats()
        self.check(self.lib.hl_b200_stats(self.h, C.byref(s)))
        return {n: int(getattr(s, n)) for n, _ in s._fields_}

    def timing_enable(self, on: bool = True) -> None:
        self.check(self.lib.hl_b200_timing_enable(self.h, 1 if on else 0))

    def timing_read(self, reset: bool = True) -> dict:
        """Device milliseconds and span counts per kernel family since the last reset (waits for the stream)."""
        t = _lib.Timing()
        self.check(self.lib.hl_b200_timing_read(self.h, C.byref(t), 1 if reset else 0))
        return {n: (float(t.ms[i]), int(t.spans[i])) for i, n in enumerate(_lib.T_NAMES)}

    def butterfly_peak(self, iters: int = 400) -> float:
        """Register-resident radix-2 butterflies per second on this device (the encoder's integer ceiling)."""
        v = C.c_double()
        self.check(self.lib.hl_b200_butterfly_peak(self.h, iters, C.byref(v)))
        return float(v.value)

    def compress_peak(self, iters: int = 400) -> float:
        """Register-resident BLAKE3 compressions per second on this device (the column hash's integer ceiling)."""
        v = C.c_double()
        self.check(self.lib.hl_b200_compress_peak(self.h, iters, C.byref(v)))
        return float(v.value)

    def lookup_inverse_table(self, alpha, g, log_len: int, d_table: int) -> None:
        """`u8_denominator_inverses` / a range family's table (protocol.rs:1125-1140) into device memory."""
        a, gg = np.array(alpha, dtype=np.uint64), np.array(g, dtype=np.uint64)
        self.check(self.lib.hl_b200_lookup_inverse_table(self.h, _ptr(a), _ptr(gg), log_len, C.c_void_p(d_table)))

    def lookup_helpers_dev(self, d_a: int, d_table_a: int, log_a: int, g_a, alpha, n: int, d_re: int, d_im: int,
                           d_b: int = 0, d_table_b: int = 0, log_b: int = 0, g_b=None) -> None:
        """One helper job (protocol.rs:1700-1800): H's two planes from one looked column or a pair, device to device."""
        al, ga = np.array(alpha, dtype=np.uint64), np.array(g_a, dtype=np.uint64)
        gb = np.array(g_b, dtype=np.uint64) if g_b is not None else None
        self.check(self.lib.hl_b200_lookup_helpers_dev(self.h, C.c_void_p(d_a), C.c_void_p(d_table_a), log_a, _ptr(ga), C.c_void_p(d_b) if d_b else None,
                                                       C.c_void_p(d_table_b) if d_b else None, log_b, _ptr(gb), _ptr(al), n, C.c_void_p(d_re), C.c_void_p(d_im)))

    def act_histogram(self, gates, outputs, f_pad: int, tokens: int, hidden: int, group_ids, tables):
        """``accuracy_act::histogram`` (accuracy_act.rs:61-79): (counts, misses)."""
        gates, outputs = np.ascontiguousarray(gates, np.int64), np.ascontiguousarray(outputs, np.int64)
        ids, tables = np.ascontiguousarray(group_ids, np.uint32), np.ascontiguousarray(tables, np.int64)
        groups = tables.size // 4096
        counts, misses = np.empty(groups * 4096, dtype=np.uint64), C.c_uint64(0)
        self.check(self.lib.hl_b200_act_histogram(self.h, _ptr(gates), _ptr(outputs), gates.size, f_pad, tokens, hidden, _ptr(ids), _ptr(tables),
                                                  groups, _ptr(counts), C.byref(misses)))
        return counts, int(misses.value)

    def act_helpers(self, gates, outputs, f_pad: int, tokens: int, hidden: int, group_ids, alpha, beta, tag) -> np.ndarray:
        """1 / ``accuracy_act::denominators`` (accuracy_act.rs:106-124, protocol.rs:993); DeviceError ERR_ZERO on a zero one."""
        gates, outputs = np.ascontiguousarray(gates, np.int64), np.ascontiguousarray(outputs, np.int64)
        ids = np.ascontiguousarray(group_ids, np.uint32)
        a, b, t = (np.array(v, dtype=np.uint64) for v in (alpha, beta, tag))
        h = np.empty((gates.size, 2), dtype=np.uint64)
        self.check(self.lib.hl_b200_act_helpers(self.h, _ptr(gates), _ptr(outputs), gates.size, f_pad, tokens, hidden, _ptr(ids), _ptr(a), _ptr(b),
                                                _ptr(t), _ptr(h)))
        return h

    def act_table(self, tables, length: int, mult, alpha, beta, tag):
        """``accuracy_act::table`` (accuracy_act.rs:13-31) and its helper m / (alpha - t) (protocol.rs:1928): (compressed, ht)."""
        tables, mult = np.ascontiguousarray(tables, np.int64), _u64(mult)
        a, b, t = (np.array(v, dtype=np.uint64) for v in (alpha, beta, tag))
        comp, ht = np.empty((length, 2), dtype=np.uint64), np.empty((length, 2), dtype=np.uint64)
        self.check(self.lib.hl_b200_act_table(self.h, _ptr(tables), tables.size // 4096, length, _ptr(mult), _ptr(a), _ptr(b), _ptr(t), _ptr(comp), _ptr(ht)))
        return comp, ht

    def witness_product(self, t_rows: int, x, xs: int, w, inner: int, outer: int, os_: int, out_len: int, in_out: bool) -> Optional[np.ndarray]:
        """``gpu::witness_product`` (metal.rs:4646-4680): the exact int16 x int8 -> int64 plane, or None when the CPU must take
        it (an activation outside int16, a shape outside the kernels' bounds)."""
        x, w = np.ascontiguousarray(x, np.int64), np.ascontiguousarray(w, np.int8)
        out, taken = np.empty(out_len, dtype=np.int64), C.c_int(0)
        self.check(self.lib.hl_b200_witness_product(self.h, t_rows, _ptr(x), x.size, xs, _ptr(w), w.size, inner, outer, os_, out_len,
                                                    1 if in_out else 0, _ptr(out), C.byref(taken)))
        return out if taken.value else None

    def witness_product_dev(self, t_rows: int, d_x: int, x_len: int, xs: int, d_w: int, w_len: int, inner: int, outer: int, os_: int, out_len: int,
                            in_out: bool, d_out: int) -> bool:
        """The same with activations, weights and the result plane resident on the device; False = not taken."""
        taken = C.c_int(0)
        self.check(self.lib.hl_b200_witness_product_dev(self.h, t_rows, C.c_void_p(d_x), x_len, xs, C.c_void_p(d_w), w_len, inner, outer, os_, out_len,
                                                        1 if in_out else 0, C.c_void_p(d_out), C.byref(taken)))
        return bool(taken.value)

    def rng_fill(self, key32: bytes, first_word: int, count: int, as_fp: bool) -> np.ndarray:
        """`count` draws of the caller's ZkRng stream (rng.rs:279-417) from word position `first_word`, expanded on the
        device: u64 words, or field elements (two words each) when `as_fp`."""
        out = np.zeros(count, dtype=np.uint64)
        self.check(self.lib.hl_b200_rng_fill(self.h, key32, first_word, count, 1 if as_fp else 0, _ptr(out)))
        return out

    def rng_fill_dev(self, key32: bytes, first_word: int, count: int, as_fp: bool, d_out: int) -> None:
        self.check(self.lib.hl_b200_rng_fill_dev(self.h, key32, first_word, count, 1 if as_fp else 0, C.c_void_p(d_out)))

    def probe_field(self, a, b) -> np.ndarray:
        """metal_probe_field: (a+b, a-b, a*b) per pair, shape (n, 3)."""
        a, b = _u64(a), _u64(b)
        out = np.empty((a.size, 3), dtype=np.uint64)
        self.check(self.lib.hl_b200_probe_field(self.h, _ptr(a), _ptr(b), a.size, _ptr(out)))
        return out

    def logup_histogram(self, idx, table_len: int) -> np.ndarray:
        """accuracy_act.rs:55-73: multiplicity of every table entry over all queries (padding included)."""
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        out = np.empty(table_len, dtype=np.uint64)
        self.check(self.lib.hl_b200_logup_histogram(self.h, _ptr(idx), idx.size, table_len, _ptr(out)))
        return out

    def logup_helpers(self, idx, outv, alpha, beta, tag, idx_off: int = 0, mult=None) -> np.ndarray:
        """protocol.rs:993-1011 / :1928: 1 / (alpha - q_i) per entry (times mult[i] when given); raises
        DeviceError with code ERR_ZERO on a zero denominator (the attempt is to be discarded)."""
        outv = np.ascontiguousarray(outv, dtype=np.int32)
        ix = np.ascontiguousarray(idx, dtype=np.int32) if idx is not None else None
        mu = _u64(mult) if mult is not None else None
        h = np.empty((outv.size, 2), dtype=np.uint64)
        a, b, t = (np.array([int(x[0]), int(x[1])], dtype=np.uint64) for x in (alpha, beta, tag))
        self.check(self.lib.hl_b200_logup_helpers(self.h, _ptr(ix), _ptr(outv), outv.size, _ptr(a), _ptr(b), _ptr(t), idx_off, _ptr(mu), _ptr(h)))
        return h

    def fold_rows_i8(self, m: np.ndarray, w: np.ndarray) -> np.ndarray:
        """mle.rs:157-185: w^T M for an int8 matrix, (cols, 2)."""
        m, w = np.ascontiguousarray(m, dtype=np.int8), _u64(w)
        out = np.empty((m.shape[1], 2), dtype=np.uint64)
        self.check(self.lib.hl_b200_fold_rows_i8(self.h, _ptr(m), m.shape[0], m.shape[1], _ptr(w), _ptr(out)))
        return out

    def fold_cols_i8(self, m: np.ndarray, c: np.ndarray) -> np.ndarray:
        """mle.rs:187-205: M c for an int8 matrix, (rows, 2)."""
        m, c = np.ascontiguousarray(m, dtype=np.int8), _u64(c)
        out = np.empty((m.shape[0], 2), dtype=np.uint64)
        self.check(self.lib.hl_b200_fold_cols_i8(self.h, _ptr(m), m.shape[0], m.shape[1], _ptr(c), _ptr(out)))
        return out

    def verify_columns(self, cols, idx, salts, paths, root: bytes, column_key: Optional[bytes], leaf_key: Optional[bytes], node_key: Optional[bytes],
                       rhos=None, wants=None, vec_store: Optional["B200Commit"] = None) -> np.ndarray:
        """The verifier's per-column checks (pcs.rs:1303-1331): cols (ncols, rows), idx (ncols,), salts (ncols, 32), paths (ncols, depth, 32).
        Returns one verdict per column: 0 accepted, 1 Merkle path fails, 2 + g disagrees with clear vector g.  What the combinations must equal
        comes as `wants` (k, ncols, 2) or as `vec_store`, the device commitment of the clear vectors' re / im rows."""
        cols, idx = _u64(cols), _u64(idx)
        ncols = idx.size
        rows = cols.size // ncols
        salts = np.ascontiguousarray(salts, dtype=np.uint8).reshape(ncols, 32)
        paths = np.ascontiguousarray(paths, dtype=np.uint8).reshape(ncols, -1, 32)
        depth = paths.shape[1]
        k = 0
        if rhos is not None:
            rhos = _u64(rhos).reshape(-1, rows, 2)
            k = rhos.shape[0]
        if wants is not None:
            wants = _u64(wants).reshape(k, ncols, 2)
        verdict = np.empty(ncols, dtype=np.int32)
        first = C.c_int64()
        self.check(self.lib.hl_b200_verify_columns(self.h, _ptr(cols), rows, ncols, _ptr(idx), _ptr(salts), _ptr(paths) if depth else None, depth, _ptr(root),
                                                   _ptr(column_key), _ptr(leaf_key), _ptr(node_key), _ptr(rhos) if k else None, k,
                                                   _ptr(wants) if wants is not None else None, vec_store.h if vec_store is not None else None,
                                                   _ptr(verdict), C.byref(first)))
        return verdict

    def merkle(self, leaves: np.ndarray, salts: Optional[np.ndarray], leaf_key: Optional[bytes], node_key: Optional[bytes]) -> np.ndarray:
        """salt_leaf_keyed + MerkleTree::build_keyed: all levels, (2 nn - 1, 32) bytes, root last."""
        leaves = np.ascontiguousarray(leaves, dtype=np.uint8)
        nn = leaves.shape[0]
        out = np.empty((2 * nn - 1, 32), dtype=np.uint8)
        s = np.ascontiguousarray(salts, dtype=np.uint8) if salts is not None else None
        self.check(self.lib.hl_b200_merkle(self.h, _ptr(leaves), _ptr(s), nn, _ptr(leaf_key), _ptr(node_key), _ptr(out)))
        return out


class B200Commit:
    """The store of a device commitment: ``impl EncodedStore`` (pcs/backend.rs:30-60)."""

    def __init__(self, ctx: Context, handle: C.c_void_p):
        self.ctx, self.h = ctx, handle
        r, n, nn, q = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_size_t()
        ctx.lib.hl_b200_store_shape(handle, C.byref(r), C.byref(n), C.byref(nn), C.byref(q))
        self.rows, self.n, self.nn, self.q = r.value, n.value, nn.value, q.value

    def fold_batch(self) -> int:
        """backend.rs:45-47: every vector in one call (the device folds in batches itself)."""
        return 1 << 30

    def fold_rows(self, rhos: np.ndarray) -> np.ndarray:
        """rho^T M over the message columns: (k, rows, 2) -> (k, n, 2)."""
        rhos = _u64(rhos)
        k = rhos.shape[0]
        out = np.empty((k, self.n, 2), dtype=np.uint64)
        self.ctx.check(self.ctx.lib.hl_b200_store_fold(self.h, _ptr(rhos), k, 0, _ptr(out)))
        return out

    def fold_rows_with_pads(self, rhos: np.ndarray) -> np.ndarray:
        """backend.rs:56-59 ([A8]): rho^T [M | pads], (k, n + q, 2); the pads are the commit's, resident."""
        rhos = _u64(rhos)
        k = rhos.shape[0]
        out = np.empty((k, self.n + self.q, 2), dtype=np.uint64)
        self.ctx.check(self.ctx.lib.hl_b200_store_fold(self.h, _ptr(rhos), k, 1, _ptr(out)))
        return out

    def columns(self, idx) -> np.ndarray:
        """The encoded columns at idx, (len(idx), rows), order of idx, duplicates repeated."""
        idx = _u64(idx)
        out = np.empty((idx.size, self.rows), dtype=np.uint64)
        self.ctx.check(self.ctx.lib.hl_b200_store_columns(self.h, _ptr(idx), idx.size, _ptr(out)))
        return out

    def merkle(self, salts: Optional[np.ndarray], leaf_key: Optional[bytes], node_key: Optional[bytes], out: Optional[np.ndarray] = None) -> np.ndarray:
        """All levels of the salted tree, (2 nn - 1, 32).  `out`: the caller's buffer for them (page-locked memory makes the read-back
        a direct copy)."""
        if out is None:
            out = np.empty((2 * self.nn - 1, 32), dtype=np.uint8)
        assert out.dtype == np.uint8 and out.size == (2 * self.nn - 1) * 32 and out.flags.c_contiguous
        s = np.ascontiguousarray(salts, dtype=np.uint8) if salts is not None else None
        self.ctx.check(self.ctx.lib.hl_b200_store_merkle(self.h, _ptr(s), _ptr(leaf_key), _ptr(node_key), _ptr(out)))
        return out

    def merkle_dev(self, d_salts: int, leaf_key: Optional[bytes], node_key: Optional[bytes], d_levels: int) -> None:
        """Salted leaves and tree, device to device, asynchronous on the context's stream."""
        self.ctx.check(self.ctx.lib.hl_b200_store_merkle_dev(self.h, C.c_void_p(d_salts), _ptr(leaf_key), _ptr(node_key), C.c_void_p(d_levels)))

    def encoded_dev(self) -> int:
        return int(self.ctx.lib.hl_b200_store_encoded_dev(self.h) or 0)

    def leaves_dev(self) -> int:
        return int(self.ctx.lib.hl_b200_store_leaves_dev(self.h) or 0)

    def free(self) -> None:
        if self.h:
            self.ctx.lib.hl_b200_store_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class B200Backend:
    """``impl Backend`` (pcs/backend.rs:66-100) for this device; the adapter's ``backend()``."""

    def __init__(self, ctx: Optional[Context] = None, device: int = 0):
        self.ctx = ctx or Context(device)

    def enabled(self) -> bool:
        return True

    def label(self) -> str:
        return self.ctx.label()

    def try_commit(self, log_cols: int, inv_rate: int, data, max_log: int, key: Optional[bytes] = None):
        data = _u64(data)
        rows = data.size >> log_cols
        leaves = np.empty((inv_rate << log_cols, 32), dtype=np.uint8)
        h = C.c_void_p()
        rc = self.ctx.lib.hl_b200_commit(self.ctx.h, log_cols, inv_rate, _ptr(data), rows, max_log, _ptr(key), C.byref(h), _ptr(leaves))
        if rc != 0:
            self.ctx.declined("b200 commit", rc)
            return None
        return B200Commit(self.ctx, h), leaves

    def try_commit_zk(self, log_cols: int, inv_rate: int, data, pads, pows, max_log: int):
        return self.try_commit_zk_keyed(log_cols, inv_rate, data, pads, pows, max_log, None)

    def try_commit_zk_keyed(self, log_cols: int, inv_rate: int, data, pads, pows, max_log: int, key: Optional[bytes], leaves_out: Optional[np.ndarray] = None):
        data, pads, pows = _u64(data), _u64(pads), _u64(pows)
        rows = data.size >> log_cols
        q = pads.size // rows if rows else 0
        leaves = leaves_out if leaves_out is not None else np.empty((inv_rate << log_cols, 32), dtype=np.uint8)
        assert leaves.dtype == np.uint8 and leaves.size == (inv_rate << log_cols) * 32 and leaves.flags.c_contiguous
        h = C.c_void_p()
        rc = self.ctx.lib.hl_b200_commit_zk(self.ctx.h, log_cols, inv_rate, _ptr(data), rows, _ptr(pads), q, _ptr(pows), max_log,
                                             _ptr(key), C.byref(h), _ptr(leaves))
        if rc != 0:
            self.ctx.declined("b200 zk commit", rc)
            return None
        return B200Commit(self.ctx, h), leaves

    def try_commit_zk_tree(self, log_cols: int, inv_rate: int, data, pads, pows, max_log: int, key: Optional[bytes], salts, leaf_key: Optional[bytes],
                           node_key: Optional[bytes], leaves_out: Optional[np.ndarray] = None, levels_out: Optional[np.ndarray] = None,
                           want_leaves: bool = True):
        """The commitment and its salted tree in one call (pcs.rs:782-817: the salts are drawn before the commitment is offered):
        (store, leaves, levels) or None on a decline.  want_leaves False: the unsalted leaves stay on the device (leaves is None)."""
        data, pads, pows = _u64(data), _u64(pads), _u64(pows)
        salts = np.ascontiguousarray(salts, dtype=np.uint8)
        rows, nn = data.size >> log_cols, inv_rate << log_cols
        q = pads.size // rows if rows else 0
        leaves = None if not want_leaves else leaves_out if leaves_out is not None else np.empty((nn, 32), dtype=np.uint8)
        levels = levels_out if levels_out is not None else np.empty((2 * nn - 1, 32), dtype=np.uint8)
        assert (leaves is None or leaves.size == nn * 32) and levels.size == (2 * nn - 1) * 32 and salts.size == nn * 32
        h = C.c_void_p()
        rc = self.ctx.lib.hl_b200_commit_zk_tree(self.ctx.h, log_cols, inv_rate, _ptr(data), rows, _ptr(pads), q, _ptr(pows), max_log, _ptr(key),
                                                  _ptr(salts), _ptr(leaf_key), _ptr(node_key), C.byref(h), _ptr(leaves), _ptr(levels))
        if rc != 0:
            self.ctx.declined("b200 zk commit with tree", rc)
            return None
        return B200Commit(self.ctx, h), leaves, levels

    def try_commit_zk_packed(self, log_cols: int, inv_rate: int, packed: np.ndarray, row_width: np.ndarray, pads, pows, max_log: int,
                             key: Optional[bytes], salts=None, leaf_key: Optional[bytes] = None, node_key: Optional[bytes] = None,
                             levels_out: Optional[np.ndarray] = None, want_leaves: bool = True):
        """The hiding commitment from packed narrow rows (`pack_rows`): (store, leaves[, levels]) or None on a decline.  The
        device restores the 64-bit image (gpu/cuda.rs:1073-1105 `upload_narrow` + `k_widen`), so every result equals the
        wide call's."""
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        row_width = np.ascontiguousarray(row_width, dtype=np.uint8)
        pads, pows = _u64(pads), _u64(pows)
        rows, nn = row_width.size, inv_rate << log_cols
        q = pads.size // rows if rows else 0
        assert packed.size == int(row_width.astype(np.int64).sum()) << log_cols
        tree = salts is not None
        leaves = np.empty((nn, 32), dtype=np.uint8) if (want_leaves or not tree) else None
        levels = None
        if tree:
            salts = np.ascontiguousarray(salts, dtype=np.uint8)
            levels = levels_out if levels_out is not None else np.empty((2 * nn - 1, 32), dtype=np.uint8)
            assert salts.size == nn * 32 and levels.size == (2 * nn - 1) * 32
        h = C.c_void_p()
        rc = self.ctx.lib.hl_b200_commit_zk_packed(self.ctx.h, log_cols, inv_rate, _ptr(packed), _ptr(row_width), rows, _ptr(pads), q, _ptr(pows), max_log,
                                                   _ptr(key), _ptr(salts) if tree else None, _ptr(leaf_key), _ptr(node_key), C.byref(h),
                                                   _ptr(leaves) if leaves is not None else None, _ptr(levels) if tree else None)
        if rc != 0:
            self.ctx.declined("b200 zk commit (packed rows)", rc)
            return None
        st = B200Commit(self.ctx, h)
        return (st, leaves, levels) if tree else (st, leaves)

    def check_opening_columns(self, log_cols: int, inv_rate: int, pows, max_log: int, cols, idx, salts, paths, root: bytes, column_key: Optional[bytes],
                              leaf_key: Optional[bytes], node_key: Optional[bytes], rhos, vecs, one_call: bool = True) -> Optional[np.ndarray]:
        """The data-parallel part of `verify_zk_tagged` (pcs.rs:1282-1331) on the device: the clear vectors (G + 1, n + q, 2) are encoded as
        2 (G + 1) base rows (re and im apart, pcs.rs:1287-1296) by the commitment's own encoder, and every opened column is hashed, walked to the
        root and compared with them.  `one_call`: through `hl_b200_verify_opening`; otherwise as the two calls a caller who keeps the vectors'
        commitment would make.  None when the device declines the shape (the caller then runs its host body)."""
        vecs = _u64(vecs)
        n = 1 << log_cols
        g1 = vecs.shape[0]
        if one_call:
            cols, idx, rhos, pows = _u64(cols), _u64(idx), _u64(rhos), _u64(pows)
            ncols = idx.size
            rows = cols.size // ncols
            salts = np.ascontiguousarray(salts, dtype=np.uint8).reshape(ncols, 32)
            paths = np.ascontiguousarray(paths, dtype=np.uint8).reshape(ncols, -1, 32)
            depth = paths.shape[1]
            verdict = np.empty(ncols, dtype=np.int32)
            first = C.c_int64()
            rc = self.ctx.lib.hl_b200_verify_opening(self.ctx.h, log_cols, inv_rate, vecs.shape[1] - n, _ptr(pows), _ptr(vecs), g1, _ptr(cols), rows, ncols, _ptr(idx),
                                                     _ptr(salts), _ptr(paths) if depth else None, depth, _ptr(root), _ptr(column_key), _ptr(leaf_key),
                                                     _ptr(node_key), _ptr(rhos), _ptr(verdict), C.byref(first))
            if rc != 0:
                self.ctx.declined("b200 verify opening", rc)
                return None
            return verdict
        planes = np.ascontiguousarray(np.moveaxis(vecs, 2, 1)).reshape(2 * g1, -1)  # row 2 g + c = component c of vector g
        got = self.try_commit_zk_keyed(log_cols, inv_rate, np.ascontiguousarray(planes[:, :n]), np.ascontiguousarray(planes[:, n:]), pows, max_log, None)
        if got is None:
            return None
        store, _ = got
        try:
            return self.ctx.verify_columns(cols, idx, salts, paths, root, column_key, leaf_key, node_key, rhos=rhos, vec_store=store)
        finally:
            store.free()

    def commit_zk_dev(self, log_cols: int, inv_rate: int, d_data: int, rows: int, d_pads: int, q: int, d_pows: int,
                      key: Optional[bytes], d_leaves: int = 0) -> B200Commit:
        """The device-buffer commitment: inputs are device addresses, asynchronous on the context's stream."""
        h = C.c_void_p()
        self.ctx.check(self.ctx.lib.hl_b200_commit_zk_dev(self.ctx.h, log_cols, inv_rate, C.c_void_p(d_data), rows, C.c_void_p(d_pads), q,
                                                            C.c_void_p(d_pows), _ptr(key), C.byref(h), C.c_void_p(d_leaves)))
        return B200Commit(self.ctx, h)


def narrow_class(words: np.ndarray) -> int:
    """The signed byte width that represents every word of `words` exactly (gpu/cuda.rs:903-910 `narrow_class`): 1, 2 or 4
    for int8 / int16 / int32 valued field words (x >= 0 stored as x, x < 0 as p + x), 8 for anything wider."""
    w = _u64(words)
    P = np.uint64(0xFFFFFFFF00000001)
    for width, hi in ((1, 0x80), (2, 0x8000), (4, 0x80000000)):
        if bool(np.all((w < np.uint64(hi)) | (w >= P - np.uint64(hi)))):
            return width
    return 8


def pack_rows(data: np.ndarray, rows: int) -> Tuple[np.ndarray, np.ndarray]:
    """(packed bytes, per-row widths) of a rows x n matrix of canonical field words for `try_commit_zk_packed`: every row
    at the narrowest width that holds it (gpu/cuda.rs:926-960 `pack_narrow`, per row instead of per upload)."""
    d = _u64(data).reshape(rows, -1)
    widths = np.array([narrow_class(d[r]) for r in range(rows)], dtype=np.uint8)
    P = np.uint64(0xFFFFFFFF00000001)
    parts = []
    for r in range(rows):
        w = int(widths[r])
        if w == 8:
            parts.append(d[r].view(np.uint8))
            continue
        with np.errstate(over="ignore"):
            signed = np.where(d[r] < np.uint64(1 << 63), d[r], d[r] - P).astype(np.uint64).view(np.int64)  # p + x -> x (mod 2^64)
        parts.append(signed.astype({1: np.int8, 2: "<i2", 4: "<i4"}[w]).view(np.uint8))
    return np.concatenate(parts), widths


class B200Mask(B200Commit):
    """``MaskCommit`` on the device (hashline/src/zk.rs:395-411, 447-536): a store whose data rows are the coefficient rows
    (a_coefs zero-extended, b_re, b_im, u_re, u_im), so the tree, the opened columns and the proximity combination are the
    store's own calls; ``open_q`` is the product polynomial of ``mask_open`` (zk.rs:623-637)."""

    def __init__(self, ctx: Context, handle: C.c_void_p, n_masks: int, a_coefs: np.ndarray, leaves: np.ndarray):
        super().__init__(ctx, handle)
        self.n_masks, self.a_coefs, self.leaves = n_masks, a_coefs, leaves

    def open_q(self, ws: np.ndarray) -> np.ndarray:
        """ws: (n_masks, m, 2) combined weights (zk.rs:553-578) -> q' (2 m, 2)."""
        ws = _u64(ws)
        q = np.empty((self.n, 2), dtype=np.uint64)
        self.ctx.check(self.ctx.lib.hl_b200_mask_open_q(self.h, self.n_masks, _ptr(ws), _ptr(q)))
        return q

    def prox(self, rs: np.ndarray) -> np.ndarray:
        """sum_row r_row p_row + u (zk.rs:641-647): rs (2 n_masks + 2, 2) -> (2 m, 2)."""
        rs = _u64(rs).reshape(-1, 2)
        w = np.concatenate([rs, np.array([[1, 0], [0, 1]], dtype=np.uint64)])  # u = u_re + U u_im
        return self.fold_rows(w.reshape(1, self.rows, 2))[0]


def mask_commit(ctx: Context, msgs: np.ndarray, coef_rows: np.ndarray, pows: np.ndarray, col_key: Optional[bytes], log_msg: int = 9, log_dom: int = 12):
    """``mask_commit[_tagged]`` (zk.rs:447-536) after its draws: msgs = the 2 S message rows (coefficients of a mask's real or
    imaginary part, its pads, zeros) as they stand before ``ntt.inverse``; coef_rows = (b_re, b_im, u_re, u_im).  Returns the
    ``B200Mask`` (``a_coefs`` and unsalted ``leaves`` on it), or None when the device declines."""
    msgs, coef_rows, pows = _u64(msgs), _u64(coef_rows), _u64(pows)
    m = 1 << log_msg
    n_msg, n_coef = msgs.size // m, coef_rows.size // (2 * m)
    a_coefs = np.empty((n_msg, m), dtype=np.uint64)
    leaves = np.empty((1 << log_dom, 32), dtype=np.uint8)
    h = C.c_void_p()
    rc = ctx.lib.hl_b200_mask_commit(ctx.h, log_msg, log_dom, _ptr(msgs), n_msg, _ptr(coef_rows), n_coef, _ptr(pows), _ptr(col_key), C.byref(h),
                                     _ptr(a_coefs), _ptr(leaves))
    if rc != 0:
        ctx.declined("b200 mask commit", rc)
        return None
    return B200Mask(ctx, h, n_msg // 2, a_coefs, leaves)


POLY_PROD, POLY_ZC, POLY_LOGUP_Q, POLY_LOGUP_T = 0, 1, 2, 3


_P = 0xFFFFFFFF00000001


def _f2_mul(a, b):
    return ((a[0] * b[0] + 7 * a[1] * b[1]) % _P, (a[0] * b[1] + a[1] * b[0]) % _P)


def eq_table_msb(point) -> np.ndarray:
    """The eq table of a point, first coordinate = most significant index bit (zkp-core/src/mle.rs:53-59): host logic of the
    table plans, small (a half point or a plane's fixed coordinates)."""
    e = [(1, 0)]
    for r in point:
        r = (int(r[0]), int(r[1]))
        one_minus = ((1 - r[0]) % _P, (-r[1]) % _P)
        e = [v for x in e for v in (_f2_mul(x, one_minus), _f2_mul(x, r))]
    return np.array(e, dtype=np.uint64).reshape(-1, 2)


def plane_maps(n_vars: int, coords):
    """The index maps of a committed plane's table, as the host builder makes them (private_block/argument.rs:486-512):
    `used` (cube variables the plane reads), the inverse bit map in two halves (cube index -> plane index, split at
    xlo = n_vars / 2), the plane-index bits of every pattern z of the fixed coordinates (first fixed coordinate = most
    significant bit of z) and the eq table of the fixed coordinates.  Coordinate j reads plane-index bit log - 1 - j."""
    n, log = n_vars, len(coords)
    bit_of, fpos, fixed = {}, [], []
    for j, c in enumerate(coords):
        if c[0] == "fixed":
            fpos.append(log - 1 - j)
            fixed.append(c[1])
        else:
            xb = n - 1 - c[1]
            if xb in bit_of:
                raise ValueError("plane_maps: a cube variable read by two coordinates (the host builder accumulates; not planned)")
            bit_of[xb] = (log - 1 - j, 1 if c[0] == "flip" else 0)
    used = sum(1 << b for b in bit_of)
    xlo = n // 2

    def inverse_half(shift, bits):
        out = np.zeros(1 << bits, dtype=np.uint32)
        v = np.arange(1 << bits, dtype=np.uint32)
        for b in range(bits):
            if shift + b in bit_of:
                ib, flip = bit_of[shift + b]
                out |= (((v >> np.uint32(b)) & np.uint32(1)) ^ np.uint32(flip)) << np.uint32(ib)
        return out

    inv_lo, inv_hi = inverse_half(0, xlo), inverse_half(xlo, n - xlo)
    nf = len(fpos)
    nz = (1 << nf) if nf else 0
    zbits = np.array([sum(((z >> (nf - 1 - t)) & 1) << fpos[t] for t in range(nf)) for z in range(nz)], dtype=np.uint32)
    eqf = eq_table_msb(fixed) if nf else None
    return used, xlo, inv_lo, inv_hi, zbits, eqf


class B200Tables:
    """A slot's tables built on the device: the mirror of the reference's `MetalTables` (gpu/metal.rs: `new`, `tables_mut`,
    `plan_eq`, `plan_plane`, `build_planned` / `flush`, `to_vecs`).  The index maps of a plane are made here, on the host,
    exactly as the host builder makes them (private_block/argument.rs:486-512); the kernels only read them."""

    def __init__(self, ctx: Context, k: int, n_vars: int):
        self.ctx, self.k, self.n_vars = ctx, k, n_vars
        h = C.c_void_p()
        ctx.check(ctx.lib.hl_b200_tables_new(ctx.h, k, n_vars, C.byref(h)))
        self.h = h

    def put(self, i: int, words: np.ndarray) -> None:
        words = _u64(words)
        assert words.size == 2 << self.n_vars
        self.ctx.check(self.ctx.lib.hl_b200_tables_put(self.h, i, _ptr(words)))

    def plan_eq(self, i: int, point, start: int, base_check: bool = False) -> None:
        """`Tab::Eq { point, start }`: eq(point, x[start .. start + |point|]) (argument.rs:643-660)"""
        point = _u64(point).reshape(-1, 2)
        p = point.shape[0]
        p_lo = p // 2
        hi, lo = eq_table_msb(point[: p - p_lo]), eq_table_msb(point[p - p_lo:])
        self.ctx.check(self.ctx.lib.hl_b200_tables_eq(self.h, i, start, p, _ptr(hi), _ptr(lo), 1 if base_check else 0))

    def plan_plane(self, i: int, rows, coords, slices, base_check: bool = False) -> None:
        """`Tab::Priv`: a committed plane (argument.rs:386-577).  `rows`: a `B200Commit` (its resident data rows) or a
        (device address, word count) pair; `coords`: the plane's coordinates, first = most significant index bit, each
        ("rho", k) | ("flip", k) | ("fixed", (c0, c1)); `slices`: [(word offset, (c0, c1))]."""
        used, xlo, inv_lo, inv_hi, zbits, eqf = plane_maps(self.n_vars, coords)
        nz = zbits.size
        sl = np.array([[off, cf[0], cf[1]] for off, cf in slices], dtype=np.uint64)
        store, d_rows, n_words = (rows.h, None, 0) if isinstance(rows, B200Commit) else (None, C.c_void_p(rows[0]), rows[1])
        self.ctx.check(self.ctx.lib.hl_b200_tables_plane(self.h, i, store, d_rows, n_words, used, xlo, _ptr(inv_lo), _ptr(inv_hi),
                                                         _ptr(zbits) if nz else None, nz, _ptr(eqf) if nz else None, _ptr(sl), sl.shape[0],
                                                         1 if base_check else 0))

    def flush(self) -> None:
        self.ctx.check(self.ctx.lib.hl_b200_tables_flush(self.h))

    def read(self, i: int) -> np.ndarray:
        out = np.zeros((1 << self.n_vars, 2), dtype=np.uint64)
        self.ctx.check(self.ctx.lib.hl_b200_tables_read(self.h, i, _ptr(out)))
        return out

    def free(self) -> None:
        if self.h:
            self.ctx.lib.hl_b200_tables_free(self.h)
            self.h = None


class SlotProgram:
    """A slot polynomial as data: the grammar of the reference's slot expression graph (private_block/slot_ir.rs:57-345:
    `TableRef`, `Node` with `NodeBody::{Affine, Sum}`, `SlotTerm`), flattened into the word stream the C ABI takes
    (include/hl_b200.h, `hl_b200_rounds_new_ir`).  Build it in the reference's order: nodes first (each refers only to
    earlier nodes), then the top-level terms.  A coefficient is `ONE`, `NEG_ONE`, `ZERO` or an Fp2 `(c0, c1)`."""

    ONE, NEG_ONE, ZERO = "one", "neg-one", "zero"
    _SPECIAL = {"one": 0xFFFFFFFF, "neg-one": 0xFFFFFFFE, "zero": 0xFFFFFFFD}
    NODE_FLAG = 0x80000000

    def __init__(self, n_tables: int):
        self.n_tables = n_tables
        self.coefs: List[Tuple[int, int]] = []
        self._coef_index = {}
        self._words: List[int] = []
        self.n_nodes = 0
        self.n_terms = 0

    @staticmethod
    def node(node_id: int) -> int:
        """the factor word of node `node_id` (a table's factor word is its id)"""
        return SlotProgram.NODE_FLAG | node_id

    def _coef(self, c) -> int:
        if isinstance(c, str):
            return self._SPECIAL[c]
        key = (int(c[0]), int(c[1]))
        # by VALUE, as the flattening of a `SlotIr` does: a coefficient equal to 1, -1 or 0 is the special word
        if key == (1, 0):
            return self._SPECIAL["one"]
        if key == (0xFFFFFFFF00000000, 0):
            return self._SPECIAL["neg-one"]
        if key == (0, 0):
            return self._SPECIAL["zero"]
        if key not in self._coef_index:
            self._coef_index[key] = len(self.coefs)
            self.coefs.append(key)
        return self._coef_index[key]

    def _product(self, coef, factors) -> None:
        self._words += [self._coef(coef), len(factors)] + [int(f) for f in factors]

    def affine(self, konst, terms) -> int:
        """`NodeBody::Affine`: konst + sum coef_i * table_i; `terms` = [(coef, table id)].  Returns the node id."""
        assert self.n_terms == 0, "nodes come before terms"
        self._words += [0 | (len(terms) << 8), self._coef(konst)]
        for c, t in terms:
            self._words += [self._coef(c), int(t)]
        self.n_nodes += 1
        return self.n_nodes - 1

    def sum(self, subterms) -> int:
        """`NodeBody::Sum`: sum coef * prod(factors); `subterms` = [(coef, [factor words])].  Returns the node id."""
        assert self.n_terms == 0, "nodes come before terms"
        self._words.append(1 | (len(subterms) << 8))
        for c, fs in subterms:
            self._product(c, fs)
        self.n_nodes += 1
        return self.n_nodes - 1

    def term(self, coef, wrapper, inner) -> None:
        """`SlotTerm`: coef * prod(wrapper tables) * prod(inner factors)"""
        self._product(coef, list(wrapper) + list(inner))
        self.n_terms += 1

    def words(self) -> np.ndarray:
        return np.array(self._words, dtype=np.uint32)

    def coef_array(self) -> np.ndarray:
        return np.array(self.coefs, dtype=np.uint64).reshape(-1, 2)


class B200Rounds:
    """``impl SumcheckRounds`` (sumcheck/rounds.rs:22-28) with the tables resident on the device, plus the
    device-side batch of rounds the reference's Metal evaluator runs (metal.rs:4141 ``masked_prove``)."""

    def __init__(self, ctx: Context, poly, tables: np.ndarray, degree: int, coefs=None):
        """`poly`: one of the POLY_* families, or a `SlotProgram` (any slot polynomial, as data).  `tables`: (k, 2^n, 2) host
        words, or a `B200Tables` set built on the device (taken over: `metal_rounds_owned`, gpu/metal.rs:2804)."""
        self._degree = degree
        h = C.c_void_p()
        if isinstance(tables, B200Tables):
            self.ctx, self.k, self._n_vars = ctx, tables.k, tables.n_vars
            if isinstance(poly, SlotProgram):
                w, cf = poly.words(), poly.coef_array()
                ctx.check(ctx.lib.hl_b200_rounds_from_tables_ir(ctx.h, degree, tables.h, w.ctypes.data_as(C.c_void_p), w.size, poly.n_nodes,
                                                                poly.n_terms, _ptr(cf) if cf.size else None, cf.shape[0], C.byref(h)))
            else:
                cf = _u64(coefs).reshape(-1, 2) if coefs is not None else None
                ctx.check(ctx.lib.hl_b200_rounds_from_tables(ctx.h, poly, degree, tables.h, _ptr(cf), 0 if cf is None else cf.shape[0], C.byref(h)))
            tables.free()
            self.h = h
            return
        tables = _u64(tables)
        assert tables.ndim == 3 and tables.shape[2] == 2
        self.ctx, self.k = ctx, tables.shape[0]
        self._n_vars = int(tables.shape[1]).bit_length() - 1
        assert tables.shape[1] == 1 << self._n_vars
        if isinstance(poly, SlotProgram):
            assert poly.n_tables == self.k
            w, cf = poly.words(), poly.coef_array()
            ctx.check(ctx.lib.hl_b200_rounds_new_ir(ctx.h, self.k, self._n_vars, degree, _ptr(tables), w.ctypes.data_as(C.c_void_p), w.size,
                                                    poly.n_nodes, poly.n_terms, _ptr(cf) if cf.size else None, cf.shape[0], C.byref(h)))
        else:
            cf = _u64(coefs).reshape(-1, 2) if coefs is not None else None
            ctx.check(ctx.lib.hl_b200_rounds_new(ctx.h, poly, self.k, self._n_vars, degree, _ptr(tables), _ptr(cf),
                                                 0 if cf is None else cf.shape[0], C.byref(h)))
        self.h = h

    def n_vars(self) -> int:
        return self._n_vars

    def degree(self) -> int:
        return self._degree

    def round(self, j: int, eval_one: bool = True) -> np.ndarray:
        out = np.zeros((self._degree + 1, 2), dtype=np.uint64)
        self.ctx.check(self.ctx.lib.hl_b200_rounds_round(self.h, j, 1 if eval_one else 0, _ptr(out)))
        return out

    def fold(self, r) -> None:
        rr = np.array([int(r[0]), int(r[1])], dtype=np.uint64)
        self.ctx.check(self.ctx.lib.hl_b200_rounds_fold(self.h, _ptr(rr)))

    def finals(self) -> np.ndarray:
        out = np.zeros((self.k, 2), dtype=np.uint64)
        self.ctx.check(self.ctx.lib.hl_b200_rounds_finals(self.h, _ptr(out)))
        return out

    def batched(self, nd: int, state: bytes, counter: int, key: Optional[bytes] = None, mask: Optional[np.ndarray] = None,
                mask_vars: int = 0, mask_c=(0, 0), recover_one: bool = False, claim=None):
        """`nd` rounds on the device from transcript position (state, counter).  Returns
        (sums (nd, D+1, 2), absorbed (nd, D+1, 2), challenges (nd, 2), new state, new counter, running claim)."""
        fs = _lib.FsState()
        C.memmove(fs.state, state, 32)
        fs.counter = counter
        if key:
            C.memmove(fs.key, key, 32)
        fs.keyed = 1 if key else 0
        fs.recover_one = 1 if recover_one else 0
        fs.have_claim = 1 if claim is not None else 0
        if claim is not None:
            fs.claim[0], fs.claim[1] = int(claim[0]), int(claim[1])
        np_ = self._degree + 1
        out = np.zeros((nd, 2 * np_ + 1, 2), dtype=np.uint64)
        mk = _u64(mask).reshape(-1, 2) if mask is not None else None
        mc = np.array([int(mask_c[0]), int(mask_c[1])], dtype=np.uint64)
        self.ctx.check(self.ctx.lib.hl_b200_rounds_batched(self.h, nd, C.byref(fs), _ptr(mk), mask_vars, _ptr(mc), _ptr(out)))
        return out[:, :np_], out[:, np_:2 * np_], out[:, 2 * np_], bytes(fs.state), int(fs.counter), (int(fs.claim[0]), int(fs.claim[1]))

    def free(self) -> None:
        if self.h:
            self.ctx.lib.hl_b200_rounds_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def hash_columns_static(d_encoded: int, rows: int, nn: int, key: Optional[bytes], d_leaves: int, cuda_stream: int = 0) -> None:
    """Column leaves of a device-resident rows x nn matrix into a device buffer, for callers that must not
    allocate device memory (a pre-carved serving loop, a plug-in inside someone else's process).  The scratch
    is a fixed 24 MiB array inside the library, so shapes with ceil(rows/128) * nn * 32 bytes above that are
    refused; the call works on the current device, is asynchronous on `cuda_stream`, and must not overlap
    another call of itself on the same GPU."""
    lib = _lib.load()
    rc = lib.hl_b200_hash_columns_static(C.c_void_p(d_encoded), rows, nn, _ptr(key), C.c_void_p(d_leaves), C.c_void_p(cuda_stream))
    if rc != 0:
        raise DeviceError(rc, "hash_columns_static: " + {-1: "bad argument", -7: "shape exceeds the 24 MiB static scratch"}.get(rc, "device error"))
