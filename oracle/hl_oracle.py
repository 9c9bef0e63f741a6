"""TEST INFRASTRUCTURE, NOT PRODUCT CODE.

ctypes front of the CPU oracle (``libhl_oracle.so``, built from the C files beside
this one) plus the small amount of host protocol logic the reference keeps around
the primitives: hash tags, the hiding commitment's draw order, claim grouping and
the opening of ``zkp-core/src/pcs.rs``.  Only the tests, the smoke check and the
bench's CPU baseline import this module.

Field elements travel as ``numpy.uint64``; an Fp2 is two consecutive words
``(c0, c1)``, so an Fp2 vector of length n is a ``(n, 2)`` uint64 array.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

P = 0xFFFFFFFF00000001
_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libhl_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the system gcc (the Makefile beside this file)."""
    srcs = [os.path.join(_HERE, f) for f in ("blake3.c", "ntt.c", "transcript.c", "sumcheck.c", "logup.c", "tables.c", "witness.c", "hl_oracle.h", "field.h")]
    if force or not os.path.exists(_SO) or any(os.path.getmtime(s) > os.path.getmtime(_SO) for s in srcs):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


def _load():
    if not os.path.exists(_SO):
        build()
    lib = C.CDLL(_SO)
    u64, sz, vp, i32, i64 = C.c_uint64, C.c_size_t, C.c_void_p, C.c_int, C.c_int64
    for name in ("or_fp_add", "or_fp_sub", "or_fp_mul", "or_fp_pow", "or_fp_from_u128"):
        getattr(lib, name).restype = u64
        getattr(lib, name).argtypes = [u64, u64]
    for name in ("or_fp_neg", "or_fp_inv", "or_fp_new"):
        getattr(lib, name).restype = u64
        getattr(lib, name).argtypes = [u64]
    lib.or_fp_from_i64.restype = u64
    lib.or_fp_from_i64.argtypes = [i64]
    lib.or_two_adic_root.restype = u64
    lib.or_two_adic_root.argtypes = [C.c_uint32]
    lib.or_tr_challenge_fp.restype = u64
    lib.or_rng_next_u64.restype = u64
    lib.or_rng_fp.restype = u64
    lib.or_num_threads.restype = i32
    return lib


_lib = _load()


def _p(a) -> C.c_void_p:
    if a is None:
        return C.c_void_p(0)
    if isinstance(a, (bytes, bytearray)):
        return bytes(a)
    assert a.flags["C_CONTIGUOUS"]
    return C.c_void_p(a.ctypes.data)


def _u64(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint64)


def num_threads() -> int:
    return int(_lib.or_num_threads())


def set_threads(n: int) -> None:
    _lib.or_set_threads(C.c_int(n))


# ----------------------------------------------------------------------------- field
def fp_add(a, b): return int(_lib.or_fp_add(a, b))
def fp_sub(a, b): return int(_lib.or_fp_sub(a, b))
def fp_mul(a, b): return int(_lib.or_fp_mul(a, b))
def fp_neg(a): return int(_lib.or_fp_neg(a))
def fp_inv(a): return int(_lib.or_fp_inv(a))
def fp_pow(a, e): return int(_lib.or_fp_pow(a, e))
def fp_new(a): return int(_lib.or_fp_new(a))
def fp_from_u128(v): return int(_lib.or_fp_from_u128((v >> 64) & (2**64 - 1), v & (2**64 - 1)))
def fp_from_i64(v): return int(_lib.or_fp_from_i64(v))
def two_adic_root(k): return int(_lib.or_two_adic_root(k))


def fp2_add(a, b): return (fp_add(a[0], b[0]), fp_add(a[1], b[1]))
def fp2_sub(a, b): return (fp_sub(a[0], b[0]), fp_sub(a[1], b[1]))
def fp2_neg(a): return (fp_neg(a[0]), fp_neg(a[1]))
def fp2_mul_base(a, b): return (fp_mul(a[0], b), fp_mul(a[1], b))
def fp2_is_zero(a): return a[0] == 0 and a[1] == 0


def fp2_mul(a, b):
    x, y, o = (C.c_uint64 * 2)(*a), (C.c_uint64 * 2)(*b), (C.c_uint64 * 2)()
    _lib.or_fp2_mul(x, y, o)
    return (int(o[0]), int(o[1]))


def fp2_inv(a):
    x, o = (C.c_uint64 * 2)(*a), (C.c_uint64 * 2)()
    _lib.or_fp2_inv(x, o)
    return (int(o[0]), int(o[1]))


def batch_inverse2(vals: np.ndarray) -> np.ndarray:
    v = _u64(vals).copy()
    _lib.or_batch_inverse2(_p(v), C.c_size_t(v.shape[0]))
    return v


# ----------------------------------------------------------------------------- blake3
def blake3(data: bytes, key: Optional[bytes] = None, outlen: int = 32) -> bytes:
    out = C.create_string_buffer(outlen)
    _lib.or_blake3(_p(key) if key else None, data, C.c_size_t(len(data)), out, C.c_size_t(outlen))
    return out.raw


def derive_key(context: bytes, material: bytes) -> bytes:
    out = C.create_string_buffer(32)
    _lib.or_blake3_derive_key(context, C.c_size_t(len(context)), material, C.c_size_t(len(material)), out)
    return out.raw


# hashtag.rs:47-53
CTX_TRANSCRIPT = b"hashline-zk-mr1 2026-09-20 fiat-shamir transcript"
CTX_COLUMN = b"hashline-zk-mr1 2026-09-20 pcs column digest"
CTX_LEAF = b"hashline-zk-mr1 2026-09-20 pcs salted merkle leaf"
CTX_NODE = b"hashline-zk-mr1 2026-09-20 pcs merkle inner node"


@dataclass(frozen=True)
class HashTag:
    """hashtag.rs:75-150: the legacy rule (no key anywhere) or one profile's four keys."""
    transcript: Optional[bytes] = None
    column: Optional[bytes] = None
    leaf: Optional[bytes] = None
    node: Optional[bytes] = None

    @staticmethod
    def legacy() -> "HashTag":
        return HashTag()

    @staticmethod
    def for_profile(profile: str) -> "HashTag":
        p = profile.encode()
        return HashTag(derive_key(CTX_TRANSCRIPT, p), derive_key(CTX_COLUMN, p), derive_key(CTX_LEAF, p), derive_key(CTX_NODE, p))


# ----------------------------------------------------------------------------- ntt / pcs primitives
def ntt_forward(a: np.ndarray, max_log: int) -> np.ndarray:
    a = _u64(a).copy()
    _lib.or_ntt_forward(_p(a), C.c_uint32(int(a.size).bit_length() - 1), C.c_uint32(max_log))
    return a


def ntt_inverse(a: np.ndarray, max_log: int) -> np.ndarray:
    a = _u64(a).copy()
    _lib.or_ntt_inverse(_p(a), C.c_uint32(int(a.size).bit_length() - 1), C.c_uint32(max_log))
    return a


def coset_powers(h: int, nn: int) -> np.ndarray:
    out = np.empty(nn, dtype=np.uint64)
    _lib.or_coset_powers(C.c_uint64(h), C.c_size_t(nn), _p(out))
    return out


def encode_row_zk(msg, pad, pows, max_log: int) -> np.ndarray:
    msg, pad, pows = _u64(msg), _u64(pad), _u64(pows)
    out = np.empty(pows.size, dtype=np.uint64)
    _lib.or_encode_row_zk(_p(msg), C.c_size_t(msg.size), _p(pad), C.c_size_t(pad.size), _p(pows), C.c_size_t(pows.size), C.c_uint32(max_log), _p(out))
    return out


def encode_rows_zk(data, rows: int, n: int, pads, q: int, pows, max_log: int) -> np.ndarray:
    data, pads, pows = _u64(data), _u64(pads), _u64(pows)
    nn = pows.size
    enc = np.empty(rows * nn, dtype=np.uint64)
    _lib.or_encode_rows_zk(_p(data), C.c_size_t(rows), C.c_size_t(n), _p(pads), C.c_size_t(q), _p(pows), C.c_size_t(nn), C.c_uint32(max_log), _p(enc))
    return enc


def encode_rows_plain(data, rows: int, n: int, nn: int, max_log: int) -> np.ndarray:
    data = _u64(data)
    enc = np.empty(rows * nn, dtype=np.uint64)
    _lib.or_encode_rows_plain(_p(data), C.c_size_t(rows), C.c_size_t(n), C.c_size_t(nn), C.c_uint32(max_log), _p(enc))
    return enc


def hash_columns(encoded, rows: int, nn: int, key: Optional[bytes] = None) -> np.ndarray:
    encoded = _u64(encoded)
    leaves = np.empty((nn, 32), dtype=np.uint8)
    _lib.or_hash_columns(_p(encoded), C.c_size_t(rows), C.c_size_t(nn), _p(key) if key else None, _p(leaves))
    return leaves


def salt_leaves(leaves: np.ndarray, salts: np.ndarray, leaf_key: Optional[bytes] = None) -> np.ndarray:
    leaves, salts = np.ascontiguousarray(leaves, np.uint8), np.ascontiguousarray(salts, np.uint8)
    out = np.empty_like(leaves)
    _lib.or_salt_leaves(_p(leaves), _p(salts), C.c_size_t(leaves.shape[0]), _p(leaf_key) if leaf_key else None, _p(out))
    return out


def merkle_build(leaves: np.ndarray, node_key: Optional[bytes] = None) -> np.ndarray:
    """All levels, flattened: nn leaves, nn/2, ..., the root last ((2 nn - 1) x 32 bytes)."""
    leaves = np.ascontiguousarray(leaves, np.uint8)
    nn = leaves.shape[0]
    out = np.empty((2 * nn - 1, 32), dtype=np.uint8)
    _lib.or_merkle_build(_p(leaves), C.c_size_t(nn), _p(node_key) if node_key else None, _p(out))
    return out


def merkle_path(levels: np.ndarray, nn: int, j: int) -> List[bytes]:
    """merkle.rs:91-100: siblings from the leaf level up."""
    out, off, w = [], 0, nn
    while w > 1:
        out.append(bytes(levels[off + (j ^ 1)]))
        off += w
        w //= 2
        j >>= 1
    return out


def merkle_verify_path(root: bytes, idx: int, leaf: bytes, path: Sequence[bytes], node_key: Optional[bytes] = None) -> bool:
    """merkle.rs:102-127."""
    cur = leaf
    for sib in path:
        cur = blake3(cur + sib if idx & 1 == 0 else sib + cur, node_key)
        idx >>= 1
    return cur == root


def fold_rows(src, rows: int, n: int, nn: int, ir: int, rhos: np.ndarray) -> np.ndarray:
    src, rhos = _u64(src), _u64(rhos)
    k = rhos.shape[0]
    out = np.empty((k, n, 2), dtype=np.uint64)
    _lib.or_fold_rows(_p(src), C.c_size_t(rows), C.c_size_t(n), C.c_size_t(nn), C.c_size_t(ir), _p(rhos), C.c_size_t(k), _p(out))
    return out


def gather_columns(encoded, rows: int, nn: int, idx) -> np.ndarray:
    encoded, idx = _u64(encoded), _u64(idx)
    out = np.empty((idx.size, rows), dtype=np.uint64)
    _lib.or_gather_columns(_p(encoded), C.c_size_t(rows), C.c_size_t(nn), _p(idx), C.c_size_t(idx.size), _p(out))
    return out


# ----------------------------------------------------------------------------- transcript / rng
class _TrStruct(C.Structure):
    _fields_ = [("state", C.c_uint8 * 32), ("counter", C.c_uint64), ("key", C.c_uint8 * 32), ("keyed", C.c_int)]


class Transcript:
    """transcript.rs:17-167 without the masker plumbing (see `sc_prove` for masked rounds)."""

    def __init__(self, domain: bytes, key: Optional[bytes] = None):
        self._t = _TrStruct()
        self.key = key
        _lib.or_tr_new(C.byref(self._t), domain, C.c_size_t(len(domain)), _p(key) if key else None)

    @staticmethod
    def from_state(state: bytes, counter: int, key: Optional[bytes] = None) -> "Transcript":
        """a transcript resumed at a recorded (state, squeeze counter), as the reference's `Transcript::clone_state` leaves one"""
        t = Transcript(b"", key)
        C.memmove(t._t.state, state, 32)
        t._t.counter = counter
        return t

    def clone(self) -> "Transcript":
        t = Transcript.__new__(Transcript)
        t._t = _TrStruct()
        C.memmove(C.byref(t._t), C.byref(self._t), C.sizeof(_TrStruct))
        t.key = self.key
        return t

    @property
    def state(self) -> bytes:
        return bytes(self._t.state)

    @property
    def counter(self) -> int:
        return int(self._t.counter)

    def absorb(self, label: bytes, data: bytes) -> None:
        _lib.or_tr_absorb(C.byref(self._t), label, C.c_size_t(len(label)), data, C.c_size_t(len(data)))

    def absorb_u64(self, label: bytes, v: int) -> None:
        self.absorb(label, int(v).to_bytes(8, "little"))

    def absorb_fp(self, label: bytes, vals) -> None:
        self.absorb(label, _u64(vals).tobytes())

    def absorb_fp2(self, label: bytes, vals) -> None:
        self.absorb(label, _u64(vals).tobytes())

    def squeeze(self) -> bytes:
        out = C.create_string_buffer(32)
        _lib.or_tr_squeeze(C.byref(self._t), out)
        return out.raw

    def challenge_fp(self) -> int:
        return int(_lib.or_tr_challenge_fp(C.byref(self._t)))

    def challenge_fp2(self) -> Tuple[int, int]:
        o = (C.c_uint64 * 2)()
        _lib.or_tr_challenge_fp2(C.byref(self._t), o)
        return (int(o[0]), int(o[1]))

    def challenge_fp2_vec(self, n: int) -> np.ndarray:
        out = np.empty((n, 2), dtype=np.uint64)
        for i in range(n):
            out[i] = self.challenge_fp2()
        return out

    def challenge_indices(self, n: int, bound: int) -> np.ndarray:
        out = np.empty(n, dtype=np.uint64)
        _lib.or_tr_challenge_indices(C.byref(self._t), C.c_size_t(n), C.c_uint64(bound), _p(out))
        return out


class _RngStruct(C.Structure):
    _fields_ = [("key", C.c_uint8 * 32), ("counter", C.c_uint64), ("buf", C.c_uint8 * 8192), ("pos", C.c_size_t)]


class ZkRng:
    """rng.rs:279-417: BLAKE3-XOF counter mode, 8 KiB blocks."""

    def __init__(self, seed: int, domain: bytes):
        self._r = _RngStruct()
        _lib.or_rng_new(C.byref(self._r), C.c_uint64(seed), domain, C.c_size_t(len(domain)))

    @property
    def key(self) -> bytes:
        return bytes(self._r.key)

    @property
    def words_consumed(self) -> int:
        """u64 words of the stream drawn so far (block counter and position, rng.rs:300-310)"""
        return (int(self._r.counter) - 1) * 1024 + int(self._r.pos) // 8 if self._r.counter else 0

    def next_u64(self) -> int:
        return int(_lib.or_rng_next_u64(C.byref(self._r)))

    def fp(self) -> int:
        return int(_lib.or_rng_fp(C.byref(self._r)))

    def fp2(self) -> Tuple[int, int]:
        a = self.fp()
        return (a, self.fp())

    def fp_vec(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.uint64)
        _lib.or_rng_fill_fp(C.byref(self._r), _p(out), C.c_size_t(n))
        return out

    def fp2_vec(self, n: int) -> np.ndarray:
        return self.fp_vec(2 * n).reshape(n, 2)

    def bytes32(self) -> bytes:
        out = C.create_string_buffer(32)
        _lib.or_rng_bytes32(C.byref(self._r), out)
        return out.raw

    def salts(self, nn: int) -> np.ndarray:
        return np.frombuffer(b"".join(self.bytes32() for _ in range(nn)), dtype=np.uint8).reshape(nn, 32).copy()


# ----------------------------------------------------------------------------- mle / sumcheck
def eq_table(r: np.ndarray) -> np.ndarray:
    r = _u64(r).reshape(-1, 2)
    out = np.empty((1 << r.shape[0], 2), dtype=np.uint64)
    _lib.or_eq_table(_p(r), C.c_size_t(r.shape[0]), _p(out))
    return out


def eq_table_msb(r: np.ndarray) -> np.ndarray:
    r = _u64(r).reshape(-1, 2)
    out = np.empty((1 << r.shape[0], 2), dtype=np.uint64)
    _lib.or_eq_table_msb(_p(r), C.c_size_t(r.shape[0]), _p(out))
    return out


def interpolate_eval(vals: np.ndarray, x) -> Tuple[int, int]:
    vals = _u64(vals).reshape(-1, 2)
    xx, o = (C.c_uint64 * 2)(*x), (C.c_uint64 * 2)()
    _lib.or_interpolate_eval(_p(vals), C.c_size_t(vals.shape[0]), xx, o)
    return (int(o[0]), int(o[1]))


def eval_mle_ext(v: np.ndarray, r: np.ndarray) -> Tuple[int, int]:
    """mle.rs:82-86."""
    eq = eq_table_msb(r)
    acc = (0, 0)
    for a, e in zip(_u64(v).reshape(-1, 2), eq):
        acc = fp2_add(acc, fp2_mul((int(e[0]), int(e[1])), (int(a[0]), int(a[1]))))
    return acc


def eval_mle_base(v: np.ndarray, r: np.ndarray) -> Tuple[int, int]:
    """mle.rs:76-80."""
    eq = eq_table_msb(r)
    acc = (0, 0)
    for a, e in zip(_u64(v), eq):
        acc = fp2_add(acc, fp2_mul_base((int(e[0]), int(e[1])), int(a)))
    return acc


def fold_rows_i8(m: np.ndarray, w: np.ndarray) -> np.ndarray:
    m = np.ascontiguousarray(m, dtype=np.int8)
    w = _u64(w)
    out = np.empty((m.shape[1], 2), dtype=np.uint64)
    _lib.or_fold_rows_i8(_p(m), C.c_size_t(m.shape[0]), C.c_size_t(m.shape[1]), _p(w), _p(out))
    return out


def fold_cols_i8(m: np.ndarray, c: np.ndarray) -> np.ndarray:
    m = np.ascontiguousarray(m, dtype=np.int8)
    c = _u64(c)
    out = np.empty((m.shape[0], 2), dtype=np.uint64)
    _lib.or_fold_cols_i8(_p(m), C.c_size_t(m.shape[0]), C.c_size_t(m.shape[1]), _p(c), _p(out))
    return out


def eq_cube(point: np.ndarray, n_vars: int, start: int) -> np.ndarray:
    """argument.rs:586-627 over eq_table_msb(point); (2^n_vars, 2)"""
    point = _u64(point).reshape(-1, 2)
    out = np.zeros((1 << n_vars, 2), dtype=np.uint64)
    _lib.or_eq_cube(_p(point), C.c_size_t(point.shape[0]), C.c_size_t(n_vars), C.c_size_t(start), _p(out))
    return out


def priv_table(coords, slices, data: np.ndarray, n_vars: int) -> np.ndarray:
    """argument.rs:386-577 priv_table_fill (walked form).  coords: list of ("rho", k) / ("flip", k) / ("fixed", (c0, c1));
    slices: list of (offset, (c0, c1)); data: the committed rows, flat."""
    kind = np.array([{"rho": 0, "flip": 1, "fixed": 2}[c[0]] for c in coords], dtype=np.int32)
    var = np.array([c[1] if c[0] != "fixed" else 0 for c in coords], dtype=np.uint32)
    fx = np.array([c[1] for c in coords if c[0] == "fixed"], dtype=np.uint64).reshape(-1, 2)
    sl = np.array([[off, cf[0], cf[1]] for off, cf in slices], dtype=np.uint64)
    data = _u64(data)
    out = np.zeros((1 << n_vars, 2), dtype=np.uint64)
    _lib.or_priv_table(_p(kind), _p(var), _p(fx) if fx.size else None, C.c_size_t(len(coords)), _p(sl), C.c_size_t(sl.shape[0]), _p(data),
                       C.c_size_t(n_vars), _p(out))
    return out


POLY_PROD, POLY_ZC, POLY_LOGUP_Q, POLY_LOGUP_T, POLY_IR = 0, 1, 2, 3, 4

_ir_keep = None


def ir_set(words: np.ndarray, n_nodes: int, n_terms: int) -> None:
    """Select the slot polynomial that poly id POLY_IR evaluates (private_block/slot_ir.rs:352-377); `words` is the
    32-bit stream documented in include/hl_b200.h."""
    global _ir_keep
    _ir_keep = np.ascontiguousarray(words, dtype=np.uint32)
    _lib.or_ir_set(_ir_keep.ctypes.data_as(C.c_void_p), C.c_size_t(n_nodes), C.c_size_t(n_terms))



def poly_eval(poly: int, vals, coefs=None) -> Tuple[int, int]:
    vals = _u64(vals).reshape(-1, 2)
    o = (C.c_uint64 * 2)()
    cf = _u64(coefs) if coefs is not None else None
    _lib.or_poly_eval(C.c_int(poly), _p(vals), C.c_size_t(vals.shape[0]), _p(cf), o)
    return (int(o[0]), int(o[1]))


def sc_round(poly: int, tables: np.ndarray, degree: int, coefs=None, eval_one: bool = True) -> np.ndarray:
    """tables: (k, len, 2); returns (degree + 1, 2)."""
    tables = _u64(tables)
    k, ln = tables.shape[0], tables.shape[1]
    out = np.zeros((degree + 1, 2), dtype=np.uint64)
    cf = _u64(coefs) if coefs is not None else None
    _lib.or_sc_round(C.c_int(poly), _p(tables), C.c_size_t(k), C.c_size_t(ln), C.c_size_t(degree), _p(cf), C.c_int(1 if eval_one else 0), _p(out))
    return out


def cfs_round(coeffs: np.ndarray, n_vars: int, degree: int, j: int, prev: np.ndarray) -> np.ndarray:
    coeffs = _u64(coeffs)
    prev = _u64(prev).reshape(-1, 2) if j else np.zeros((1, 2), dtype=np.uint64)
    out = np.empty((degree + 1, 2), dtype=np.uint64)
    _lib.or_cfs_round(_p(coeffs), C.c_size_t(n_vars), C.c_size_t(degree), C.c_size_t(j), _p(prev), _p(out))
    return out


def cfs_total(coeffs: np.ndarray, n_vars: int, degree: int) -> Tuple[int, int]:
    coeffs, o = _u64(coeffs), (C.c_uint64 * 2)()
    _lib.or_cfs_total(_p(coeffs), C.c_size_t(n_vars), C.c_size_t(degree), o)
    return (int(o[0]), int(o[1]))


def cfs_eval(coeffs: np.ndarray, n_vars: int, degree: int, rho: np.ndarray) -> Tuple[int, int]:
    coeffs, rho, o = _u64(coeffs), _u64(rho), (C.c_uint64 * 2)()
    _lib.or_cfs_eval(_p(coeffs), C.c_size_t(n_vars), C.c_size_t(degree), _p(rho), o)
    return (int(o[0]), int(o[1]))


@dataclass
class ScOutput:
    rounds: np.ndarray      # (n, degree+1, 2) unmasked
    masked: np.ndarray      # (n, degree+1, 2) what the transcript absorbed
    challenges: np.ndarray  # (n, 2)
    finals: np.ndarray      # (k, 2)


def sc_prove(poly: int, tables: np.ndarray, degree: int, tr: Transcript, coefs=None, mask: Optional[np.ndarray] = None,
             mask_c=None, mask_vars: Optional[int] = None, recover_one: bool = False, claim=None) -> ScOutput:
    """sumcheck/rounds.rs:33-48 driver (with sumcheck.rs:282-299 masking when `mask` is given)."""
    tables = _u64(tables).copy()
    k, ln = tables.shape[0], tables.shape[1]
    n = ln.bit_length() - 1
    w = degree + 1
    rounds = np.zeros((max(n, 1), w, 2), dtype=np.uint64)
    masked = np.zeros((max(n, 1), w, 2), dtype=np.uint64)
    chal = np.zeros((max(n, 1), 2), dtype=np.uint64)
    finals = np.zeros((k, 2), dtype=np.uint64)
    cf = _u64(coefs) if coefs is not None else None
    mk = _u64(mask) if mask is not None else None
    mc = (C.c_uint64 * 2)(*(mask_c if mask_c is not None else (0, 0)))
    cl = (C.c_uint64 * 2)(*claim) if claim is not None else None
    _lib.or_sc_prove(C.c_int(poly), _p(tables), C.c_size_t(k), C.c_size_t(n), C.c_size_t(degree), _p(cf), _p(mk), mc,
                     C.c_size_t(mask_vars if mask_vars is not None else n), C.c_int(1 if recover_one else 0), cl, C.byref(tr._t),
                     _p(rounds), _p(masked), _p(chal), _p(finals))
    return ScOutput(rounds[:n], masked[:n], chal[:n], finals)


def extension_round(poly: int, finals: np.ndarray, exts: np.ndarray, degree: int, coefs=None) -> np.ndarray:
    """sumcheck.rs:302-314: s_k(X) = poly((1 - X) fin_t + X ext_t) at X = 0..=degree."""
    out = np.empty((degree + 1, 2), dtype=np.uint64)
    for x in range(degree + 1):
        v = [fp2_add(tuple(map(int, f)), fp2_mul((x, 0), fp2_sub(tuple(map(int, e)), tuple(map(int, f))))) for f, e in zip(finals, exts)]
        out[x] = poly_eval(poly, np.array(v, dtype=np.uint64), coefs)
    return out


def sc_verify(claimed, degree: int, n_rounds: int, rounds: Sequence[np.ndarray], tr: Transcript):
    """sumcheck.rs:140-165.  Returns ((final claim, challenges), None) or (None, error text)."""
    if len(rounds) != n_rounds:
        return None, f"sumcheck: expected {n_rounds} rounds, got {len(rounds)}"
    claim, chal = tuple(claimed), []
    for j, s in enumerate(rounds):
        s = _u64(s).reshape(-1, 2)
        if s.shape[0] != degree + 1:
            return None, f"sumcheck round {j}: expected degree {degree}, got {s.shape[0]} values"
        if fp2_add(tuple(map(int, s[0])), tuple(map(int, s[1]))) != claim:
            return None, f"sumcheck round {j}: s(0) + s(1) != claim"
        tr.absorb_fp2(b"sc-round", s)
        r = tr.challenge_fp2()
        chal.append(r)
        claim = interpolate_eval(s, r)
    return (claim, chal), None


# ----------------------------------------------------------------------------- logup
def logup_histogram(idx: np.ndarray, table_len: int) -> np.ndarray:
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    out = np.empty(table_len, dtype=np.uint64)
    _lib.or_logup_histogram(_p(idx), C.c_size_t(idx.size), C.c_size_t(table_len), _p(out))
    return out


def logup_helpers(idx, outv, alpha, beta, tag, idx_off: int = 0) -> np.ndarray:
    idx, outv = np.ascontiguousarray(idx, np.int32), np.ascontiguousarray(outv, np.int32)
    h = np.empty((idx.size, 2), dtype=np.uint64)
    _lib.or_logup_helpers(_p(idx), _p(outv), C.c_size_t(idx.size), (C.c_uint64 * 2)(*alpha), (C.c_uint64 * 2)(*beta),
                          (C.c_uint64 * 2)(*tag), C.c_int64(idx_off), _p(h))
    return h


def lookup_inverse_table(alpha, g, length: int):
    """protocol.rs:1125-1140: (table (length, 2) u64, absent (length,) u8)."""
    table, absent = np.zeros((length, 2), dtype=np.uint64), np.zeros(length, dtype=np.uint8)
    _lib.or_lookup_inverse_table((C.c_uint64 * 2)(*alpha), (C.c_uint64 * 2)(*g), C.c_size_t(length), _p(table), _p(absent))
    return table, absent


def lookup_helpers(a, tab_a, g_a, alpha, b=None, tab_b=None, g_b=None):
    """protocol.rs:1186-1216: (re, im) planes of one helper job, or None for "zero LogUp denominator"."""
    a = np.ascontiguousarray(a, np.int64)
    re, im = np.zeros(a.size, dtype=np.uint64), np.zeros(a.size, dtype=np.uint64)
    if b is not None:
        b = np.ascontiguousarray(b, np.int64)
        assert b.size == a.size
    tb = tab_b if b is not None else tab_a
    gb = g_b if b is not None else g_a
    _lib.or_lookup_helpers.restype = C.c_int
    bad = _lib.or_lookup_helpers(_p(a), _p(tab_a[0]), _p(tab_a[1]), C.c_size_t(tab_a[1].size), (C.c_uint64 * 2)(*g_a),
                                 _p(b) if b is not None else None, _p(tb[0]), _p(tb[1]), C.c_size_t(tb[1].size), (C.c_uint64 * 2)(*gb),
                                 (C.c_uint64 * 2)(*alpha), C.c_size_t(a.size), _p(re), _p(im))
    return None if bad else (re, im)


def act_histogram(gates, outputs, f_pad: int, tokens: int, hidden: int, group_ids, tables):
    """accuracy_act.rs:61-79: (counts (groups * 4096,), misses)."""
    gates, outputs = np.ascontiguousarray(gates, np.int64), np.ascontiguousarray(outputs, np.int64)
    ids, tables = np.ascontiguousarray(group_ids, np.uint32), np.ascontiguousarray(tables, np.int64)
    groups = tables.size // 4096
    counts = np.empty(groups * 4096, dtype=np.uint64)
    _lib.or_act_histogram.restype = C.c_uint64
    misses = _lib.or_act_histogram(_p(gates), _p(outputs), C.c_size_t(gates.size), C.c_size_t(f_pad), C.c_size_t(tokens), C.c_size_t(hidden),
                                   _p(ids), _p(tables), C.c_size_t(groups), _p(counts))
    return counts, int(misses)


def act_query_values(gates, outputs, f_pad: int, tokens: int, hidden: int, group_ids, beta, tag) -> np.ndarray:
    """accuracy_act.rs:88-95"""
    gates, outputs = np.ascontiguousarray(gates, np.int64), np.ascontiguousarray(outputs, np.int64)
    ids = np.ascontiguousarray(group_ids, np.uint32)
    q = np.empty((gates.size, 2), dtype=np.uint64)
    _lib.or_act_query_values(_p(gates), _p(outputs), C.c_size_t(gates.size), C.c_size_t(f_pad), C.c_size_t(tokens), C.c_size_t(hidden), _p(ids),
                             (C.c_uint64 * 2)(*beta), (C.c_uint64 * 2)(*tag), _p(q))
    return q


def act_helpers(gates, outputs, f_pad: int, tokens: int, hidden: int, group_ids, alpha, beta, tag):
    """denominators (accuracy_act.rs:106-124) then protocol.rs:993 inverses; None = "zero LogUp denominator"."""
    q = act_query_values(gates, outputs, f_pad, tokens, hidden, group_ids, beta, tag).astype(object)
    den = np.stack([(int(alpha[0]) - q[:, 0]) % _P0, (int(alpha[1]) - q[:, 1]) % _P0], axis=1).astype(np.uint64)
    if ((den[:, 0] | den[:, 1]) == 0).any():
        return None
    return batch_inverse2(den)


def act_table(tables, length: int, beta, tag):
    """accuracy_act.rs:13-31: (compressed (length, 2), support (length, 2))."""
    tables = np.ascontiguousarray(tables, np.int64)
    comp, sup = np.empty((length, 2), dtype=np.uint64), np.empty((length, 2), dtype=np.uint64)
    _lib.or_act_table(_p(tables), C.c_size_t(tables.size // 4096), C.c_size_t(length), (C.c_uint64 * 2)(*beta), (C.c_uint64 * 2)(*tag), _p(comp), _p(sup))
    return comp, sup


_P0 = 0xFFFFFFFF00000001


def logup_table_helper(table_out, mult, alpha, beta, tag) -> np.ndarray:
    table_out, mult = np.ascontiguousarray(table_out, np.int32), _u64(mult)
    ht = np.empty((table_out.size, 2), dtype=np.uint64)
    _lib.or_logup_table_helper(_p(table_out), _p(mult), C.c_size_t(table_out.size), (C.c_uint64 * 2)(*alpha),
                               (C.c_uint64 * 2)(*beta), (C.c_uint64 * 2)(*tag), _p(ht))
    return ht


def logup_query_values(idx, outv, beta, tag, idx_off: int = 0) -> np.ndarray:
    """accuracy_act.rs:91-99; idx None means idx_i = i (the table side)."""
    outv = np.ascontiguousarray(outv, np.int32)
    ix = np.ascontiguousarray(idx, np.int32) if idx is not None else None
    q = np.empty((outv.size, 2), dtype=np.uint64)
    _lib.or_logup_query_values(_p(ix), _p(outv), C.c_size_t(outv.size), (C.c_uint64 * 2)(*beta), (C.c_uint64 * 2)(*tag), C.c_int64(idx_off), _p(q))
    return q


def fp2_sum(v) -> Tuple[int, int]:
    v, o = _u64(v), (C.c_uint64 * 2)()
    _lib.or_fp2_sum(_p(v), C.c_size_t(v.size // 2), o)
    return (int(o[0]), int(o[1]))


# ----------------------------------------------------------------------------- the hiding commitment and its opening
@dataclass
class PcsParams:
    log_cols: int
    inv_rate: int
    num_col_checks: int

    @property
    def cols(self) -> int:
        return 1 << self.log_cols

    @property
    def enc_cols(self) -> int:
        return self.cols * self.inv_rate


@dataclass
class CommittedZk:
    """pcs.rs:607-620 (CommittedZk) with a host store."""
    params: PcsParams
    rows: int
    q: int
    data: np.ndarray       # rows*n
    pads: np.ndarray       # rows*q
    salts: np.ndarray      # nn x 32
    encoded: np.ndarray    # rows*nn
    leaves: np.ndarray     # nn x 32, unsalted
    levels: np.ndarray     # (2nn-1) x 32
    mask_rows: List[int] = field(default_factory=list)
    prox_mask_row: Optional[int] = None

    @property
    def root(self) -> bytes:
        return bytes(self.levels[-1])


def commit_zk(params: PcsParams, data: np.ndarray, max_log: int, q: int, rng: ZkRng, tag: HashTag, coset: int = 7) -> CommittedZk:
    """pcs.rs:782-817: pads (rows*q) then salts (nn) drawn in that order, then encode, hash, salt, tree."""
    data = _u64(data)
    n, nn = params.cols, params.enc_cols
    rows = data.size // n
    pads = rng.fp_vec(rows * q)
    salts = rng.salts(nn)
    pows = coset_powers(coset, nn)
    enc = encode_rows_zk(data, rows, n, pads, q, pows, max_log)
    leaves = hash_columns(enc, rows, nn, tag.column)
    levels = merkle_build(salt_leaves(leaves, salts, tag.leaf), tag.node)
    return CommittedZk(params, rows, q, data, pads, salts, enc, leaves, levels)


@dataclass
class ZPart:
    offset: int
    log_size: int
    coef: Tuple[int, int]
    point: np.ndarray  # (m, 2), possibly empty


@dataclass
class ZClaim:
    parts: List[ZPart]
    value: Tuple[int, int]


def _zpart_weights(p: ZPart, rows: int, log_cols: int):
    """pcs.rs:851-891."""
    n = 1 << log_cols
    row_w = [(0, 0)] * rows
    ls = p.log_size
    pt = _u64(p.point).reshape(-1, 2)
    if pt.shape[0] == 0:
        if ls >= log_cols:
            r0 = p.offset // n
            for i in range(1 << (ls - log_cols)):
                row_w[r0 + i] = fp2_add(row_w[r0 + i], p.coef)
            key = (b"", 0, n)
        else:
            r0, c0 = p.offset // n, p.offset % n
            row_w[r0] = fp2_add(row_w[r0], p.coef)
            key = (b"", c0, 1 << ls)
    else:
        assert pt.shape[0] == ls
        if ls >= log_cols:
            lr = ls - log_cols
            r0 = p.offset // n
            eq_r = eq_table_msb(pt[:lr])
            for i, e in enumerate(eq_r):
                row_w[r0 + i] = fp2_add(row_w[r0 + i], fp2_mul(p.coef, (int(e[0]), int(e[1]))))
            key = (pt[lr:].tobytes(), 0, n)
        else:
            r0, c0 = p.offset // n, p.offset % n
            row_w[r0] = fp2_add(row_w[r0], p.coef)
            key = (pt.tobytes(), c0, 1 << ls)
    return row_w, key


def group_zclaims(claims: Sequence[ZClaim], rows: int, log_cols: int):
    """pcs.rs:926-948: groups in first-seen order of the column key; returns [(key, [(row_w, value)])]."""
    keys, groups = [], []
    for c in claims:
        rw, key = _zpart_weights(c.parts[0], rows, log_cols)
        for p in c.parts[1:]:
            rw2, key2 = _zpart_weights(p, rows, log_cols)
            assert key2 == key
            rw = [fp2_add(a, b) for a, b in zip(rw, rw2)]
        if key in keys:
            groups[keys.index(key)][1].append((rw, c.value))
        else:
            keys.append(key)
            groups.append((key, [(rw, c.value)]))
    return groups


def zk_rhos(groups, rows: int, tr: Transcript) -> np.ndarray:
    """pcs.rs:952-973: lambdas per group, then `rows` proximity challenges.  Returns (G+1, rows, 2)."""
    out = np.zeros((len(groups) + 1, rows, 2), dtype=np.uint64)
    for g, (_, members) in enumerate(groups):
        lambdas = tr.challenge_fp2_vec(len(members))
        rho = [(0, 0)] * rows
        for (rw, _val), lam in zip(members, lambdas):
            lam = (int(lam[0]), int(lam[1]))
            for i in range(rows):
                if not fp2_is_zero(rw[i]):
                    rho[i] = fp2_add(rho[i], fp2_mul(lam, rw[i]))
        out[g] = np.array(rho, dtype=np.uint64)
    out[-1] = tr.challenge_fp2_vec(rows)
    return out


@dataclass
class OpeningZk:
    group_vecs: np.ndarray                        # (G, n+q, 2)
    prox_vec: np.ndarray                          # (n+q, 2)
    columns: List[Tuple[int, np.ndarray, bytes, List[bytes]]]

    def to_bytes(self) -> bytes:
        """pcs.rs:638-657 (OpeningZk::write_bytes)."""
        out = [self.group_vecs.tobytes(), self.prox_vec.tobytes()]
        for j, col, salt, path in self.columns:
            out.append(int(j).to_bytes(8, "little") + _u64(col).tobytes() + salt + b"".join(path))
        return b"".join(out)


def open_zk(cmz: CommittedZk, claims: Sequence[ZClaim], tr: Transcript, fold=None, columns=None) -> OpeningZk:
    """pcs.rs:1040-1069.  `fold(rhos) -> (G+1, n+q, 2)` and `columns(idx) -> (len(idx), rows)` default to the
    host store; a device store under test is plugged in through them."""
    p, rows, q = cmz.params, cmz.rows, cmz.q
    n, nn = p.cols, p.enc_cols
    groups = group_zclaims(claims, rows, p.log_cols)
    rhos = zk_rhos(groups, rows, tr)
    if fold is None:
        msg = fold_rows(cmz.data, rows, n, n, 1, rhos)
        padf = fold_rows(cmz.pads, rows, q, q, 1, rhos)
        vecs = np.concatenate([msg, padf], axis=1)
    else:
        vecs = fold(rhos)
    for v in vecs[:-1]:
        tr.absorb_fp2(b"pcs-vec", v)
    tr.absorb_fp2(b"pcs-prox", vecs[-1])
    idx = tr.challenge_indices(p.num_col_checks, nn)
    cols = gather_columns(cmz.encoded, rows, nn, idx) if columns is None else columns(idx)
    out = [(int(j), cols[c], bytes(cmz.salts[int(j)]), merkle_path(cmz.levels, nn, int(j))) for c, j in enumerate(idx)]
    return OpeningZk(vecs[:-1], vecs[-1], out)


def zkey_weights(key, log_cols: int) -> np.ndarray:
    """pcs.rs:908-920: the column weights of a group key (tail bytes, c0, len), (n, 2)."""
    tail, c0, ln = key
    out = np.zeros((1 << log_cols, 2), dtype=np.uint64)
    if len(tail) == 0:
        out[c0:c0 + ln, 0] = 1
    else:
        out[c0:c0 + ln] = eq_table_msb(np.frombuffer(tail, dtype=np.uint64).reshape(-1, 2))
    return out


def check_columns_host(cols, idx, salts, paths, root, tag, rhos, encoded_vecs) -> List[int]:
    """The body of the verifier's map over the opened columns (pcs.rs:1303-1331): per column 0 when every check holds,
    1 when the Merkle path fails, 2 + g when the column disagrees with clear vector g.  encoded_vecs: (G+1, 2, nn)."""
    out = []
    for c, j in enumerate(idx):
        col = _u64(cols[c])
        leaf = salt_leaves(hash_columns(col, col.size, 1, tag.column), np.frombuffer(salts[c], np.uint8).reshape(1, 32), tag.leaf)
        if not merkle_verify_path(root, int(j), bytes(leaf[0]), paths[c], tag.node):
            out.append(1)
            continue
        acc = fold_rows(col, col.size, 1, 1, 1, rhos)  # a26_combine, one column
        v = 0
        for g in range(rhos.shape[0]):
            if (int(acc[g, 0, 0]), int(acc[g, 0, 1])) != (int(encoded_vecs[g][0][int(j)]), int(encoded_vecs[g][1][int(j)])):
                v = 2 + g
                break
        out.append(v)
    return out


def verify_zk(params: PcsParams, q: int, root: bytes, rows: int, claims: Sequence[ZClaim], opening: OpeningZk, tr: Transcript, tag: HashTag,
              max_log: int, coset: int = 7, check_columns=None) -> Optional[str]:
    """pcs.rs:1235-1336 (`verify_zk_tagged`): None when the opening is accepted, else the reference's refusal text.
    `check_columns(cols, idx, salts, paths, root, tag, rhos, vecs, encoded_vecs) -> verdicts` defaults to the host body;
    a device verifier under test is plugged in through it (vecs: the clear vectors (G+1, n+q, 2))."""
    n, nn = params.cols, params.enc_cols
    if q < params.num_col_checks:
        return "pcs zk: fewer pads than column checks"
    depth = nn.bit_length() - 1
    for at, (_, _, _, path) in enumerate(opening.columns):
        if len(path) != depth:
            return f"pcs zk: opened column {at} carries a Merkle path of {len(path)} entries; this commitment's tree is {depth} deep"
    groups = group_zclaims(claims, rows, params.log_cols)
    if len(opening.group_vecs) != len(groups):
        return f"pcs zk: {len(opening.group_vecs)} group vectors for {len(groups)} groups"
    # zk_rhos (pcs.rs:952-973) with the combined claims
    rhos = np.zeros((len(groups) + 1, rows, 2), dtype=np.uint64)
    wants = []
    for g, (_, members) in enumerate(groups):
        lambdas = tr.challenge_fp2_vec(len(members))
        rho, want = [(0, 0)] * rows, (0, 0)
        for (rw, val), lam in zip(members, lambdas):
            lam = (int(lam[0]), int(lam[1]))
            for i in range(rows):
                if not fp2_is_zero(rw[i]):
                    rho[i] = fp2_add(rho[i], fp2_mul(lam, rw[i]))
            want = fp2_add(want, fp2_mul(lam, val))
        rhos[g] = np.array(rho, dtype=np.uint64)
        wants.append(want)
    rhos[-1] = tr.challenge_fp2_vec(rows)
    for g, (key, _) in enumerate(groups):
        v = _u64(opening.group_vecs[g]).reshape(-1, 2)
        if v.shape[0] != n + q:
            return f"pcs zk: group vector {g} has length {v.shape[0]}"
        cw = zkey_weights(key, params.log_cols)
        got = (0, 0)
        for x, y in zip(v[:n], cw):
            if int(y[0]) | int(y[1]):
                got = fp2_add(got, fp2_mul((int(x[0]), int(x[1])), (int(y[0]), int(y[1]))))
        if got != wants[g]:
            return f"pcs zk: group {g}: <v, c> != combined claim"
    for v in opening.group_vecs:
        tr.absorb_fp2(b"pcs-vec", v)
    if _u64(opening.prox_vec).reshape(-1, 2).shape[0] != n + q:
        return "pcs zk: prox vector length"
    tr.absorb_fp2(b"pcs-prox", opening.prox_vec)
    idx = tr.challenge_indices(params.num_col_checks, nn)
    if len(opening.columns) != len(idx):
        return "pcs zk: wrong number of columns"
    pows = coset_powers(coset, nn)
    vecs = np.concatenate([_u64(opening.group_vecs).reshape(-1, n + q, 2), _u64(opening.prox_vec).reshape(1, n + q, 2)], axis=0)
    encoded_vecs = [(encode_row_zk(v[:n, 0], v[n:, 0], pows, max_log), encode_row_zk(v[:n, 1], v[n:, 1], pows, max_log)) for v in vecs]
    # the map over the columns reports the first failing column, whatever its failure (pcs.rs:1303-1335)
    early = []
    for (j, col, _, _), want_j in zip(opening.columns, idx):
        if int(j) != int(want_j):
            early.append(f"pcs zk: column index {j} != sampled {int(want_j)}")
        elif len(col) != rows:
            early.append("pcs zk: column length")
        else:
            early.append(None)
    live = [c for c, e in enumerate(early) if e is None]
    cols = [opening.columns[c][1] for c in live]
    salts = [opening.columns[c][2] for c in live]
    paths = [opening.columns[c][3] for c in live]
    lidx = np.array([int(idx[c]) for c in live], dtype=np.uint64)
    if not live:
        verdicts = []
    elif check_columns is None:
        verdicts = check_columns_host(cols, lidx, salts, paths, root, tag, rhos, encoded_vecs)
    else:
        verdicts = check_columns(cols, lidx, salts, paths, root, tag, rhos, vecs, encoded_vecs)
    by_col = dict(zip(live, verdicts))
    for c, (j, _, _, _) in enumerate(opening.columns):
        if early[c] is not None:
            return early[c]
        v = by_col[c]
        if v == 1:
            return f"pcs zk: Merkle path for column {j} fails"
        if v >= 2:
            return f"pcs zk: column {j} disagrees with clear vector {v - 2}"
    return None


# ----------------------------------------------------------------------------- the masking commitment M (hashline/src/zk.rs)
# Parity of this part is UNPINNED: the reference tree holds no golden vector of an M commitment or opening (its L10 corpus is
# present only as a checksum).  Every primitive below IS pinned (transforms by the encode conformance vectors, hashing and
# trees by the L5 corpus, the generator and CfsMask::random by L5 / L6), and the restated verifier accepts the restated prover.
MASK_LOG_MSG, MASK_LOG_DOM, MASK_Q = 9, 12, 256  # zk.rs:391-393
_P = 0xFFFFFFFF00000001


def _mulp(a, b) -> np.ndarray:
    return ((_u64(a).astype(object) * _u64(b).astype(object)) % _P).astype(np.uint64)


def _addp(a, b) -> np.ndarray:
    return ((_u64(a).astype(object) + _u64(b).astype(object)) % _P).astype(np.uint64)


def encode_coeffs_coset(coeffs, pows, log_dom: int) -> np.ndarray:
    """zk.rs:441-445"""
    out = np.zeros(1 << log_dom, dtype=np.uint64)
    out[:len(coeffs)] = _mulp(coeffs, pows[:len(coeffs)])
    return ntt_forward(out, log_dom)


@dataclass
class MaskCommit:
    specs: list
    masks: list       # per spec: (n d + 2, 2) coefficients of the CFS mask
    a_coefs: np.ndarray  # 2 S x m
    encoded: np.ndarray  # (2 S + 4) x dom
    b: tuple
    u: tuple
    salts: np.ndarray
    levels: np.ndarray
    msgs: np.ndarray  # 2 S x m: the message rows before the inverse transform (what a device commit is handed)

    @property
    def root(self) -> bytes:
        return bytes(self.levels[-1])


def mask_commit(specs, rng: "ZkRng", tag: "HashTag" = None, log_msg: int = MASK_LOG_MSG, log_dom: int = MASK_LOG_DOM, q: int = MASK_Q) -> MaskCommit:
    """zk.rs:447-487 (mask_commit) / :499-536 (mask_commit_tagged): the draws in the reference's order."""
    tag = tag or HashTag.legacy()
    m, dom = 1 << log_msg, 1 << log_dom
    pows = coset_powers(7, dom)
    masks = [rng.fp2_vec(n * d + 2) for n, d in specs]  # CfsMask::random
    n_base = 2 * len(masks) + 4
    encoded = np.zeros((n_base, dom), dtype=np.uint64)
    a_coefs, msgs = [], []
    for s, mk in enumerate(masks):
        for k in range(2):
            part = mk[:, k]
            assert len(part) + q <= m
            msg = np.zeros(m, dtype=np.uint64)
            msg[:len(part)] = part
            msg[len(part):len(part) + q] = rng.fp_vec(q)
            msgs.append(msg)
            c = ntt_inverse(msg, log_dom)
            encoded[2 * s + k] = encode_coeffs_coset(c, pows, log_dom)
            a_coefs.append(c)
    b_re, b_im = rng.fp_vec(2 * m), rng.fp_vec(2 * m)
    b_re[m], b_im[m] = fp_neg(int(b_re[0])), fp_neg(int(b_im[0]))
    u_re, u_im = rng.fp_vec(2 * m), rng.fp_vec(2 * m)
    for k, c in enumerate((b_re, b_im, u_re, u_im)):
        encoded[2 * len(masks) + k] = encode_coeffs_coset(c, pows, log_dom)
    salts = rng.salts(dom)
    leaves = hash_columns(encoded, n_base, dom, tag.column)
    levels = merkle_build(salt_leaves(leaves, salts, tag.leaf), tag.node)
    return MaskCommit(list(specs), masks, np.array(a_coefs), encoded, (b_re, b_im), (u_re, u_im), salts, levels, np.array(msgs))


def mask_combined_weights(specs, functionals, theta, m: int):
    """zk.rs:553-578: functional i weighted by theta^(i+1).  functionals: [(value, [(row, weights (l, 2))])]."""
    ws = np.zeros((len(specs), m, 2), dtype=np.uint64)
    v, th = (0, 0), theta
    for value, terms in functionals:
        for row, w in terms:
            assert len(w) == specs[row][0] * specs[row][1] + 2
            for j, x in enumerate(w):
                ws[row, j] = fp2_add(tuple(int(t) for t in ws[row, j]), fp2_mul(th, (int(x[0]), int(x[1]))))
        v = fp2_add(v, fp2_mul(th, value))
        th = fp2_mul(th, theta)
    return ws, v


def _poly_mul(a, b, log_m: int) -> np.ndarray:
    """zk.rs:605-616 (poly_mul_512)"""
    m2 = 2 << log_m
    ea, eb = np.zeros(m2, dtype=np.uint64), np.zeros(m2, dtype=np.uint64)
    ea[:len(a)], eb[:len(b)] = a, b
    return ntt_inverse(_mulp(ntt_forward(ea, log_m + 1), ntt_forward(eb, log_m + 1)), log_m + 1)


def mask_open(mc: MaskCommit, functionals, tr: "Transcript", log_msg: int = MASK_LOG_MSG, log_dom: int = MASK_LOG_DOM, q: int = MASK_Q):
    """zk.rs:618-656: (q', prox, [(j, column, salt, path)]); the intermediate weights are returned as a fourth item."""
    m, dom, S = 1 << log_msg, 1 << log_dom, len(mc.masks)
    theta = tr.challenge_fp2()
    ws, _ = mask_combined_weights(mc.specs, functionals, theta, m)
    q_re, q_im = mc.b[0].copy(), mc.b[1].copy()
    seven = np.full(2 * m, 7, dtype=np.uint64)
    for s in range(S):
        w_re, w_im = ntt_inverse(ws[s, :, 0], log_dom), ntt_inverse(ws[s, :, 1], log_dom)  # weight_polys
        a_re, a_im = mc.a_coefs[2 * s], mc.a_coefs[2 * s + 1]
        rr, ii = _poly_mul(a_re, w_re, log_msg), _poly_mul(a_im, w_im, log_msg)
        ri, ir = _poly_mul(a_re, w_im, log_msg), _poly_mul(a_im, w_re, log_msg)
        q_re = _addp(_addp(q_re, rr), _mulp(ii, seven))
        q_im = _addp(_addp(q_im, ri), ir)
    qv = np.stack([q_re, q_im], axis=1)
    tr.absorb_fp2(b"mask-q", qv)
    rs = tr.challenge_fp2_vec(2 * S + 2)
    prox = np.stack([mc.u[0], mc.u[1]], axis=1).astype(object)
    for row in range(2 * S + 2):
        coeffs = mc.a_coefs[row] if row < 2 * S else mc.b[row - 2 * S]
        c = _u64(coeffs).astype(object)
        prox[:len(c), 0] = (prox[:len(c), 0] + int(rs[row, 0]) * c) % _P
        prox[:len(c), 1] = (prox[:len(c), 1] + int(rs[row, 1]) * c) % _P
    prox = prox.astype(np.uint64)
    tr.absorb_fp2(b"mask-prox", prox)
    idx = tr.challenge_indices(q, dom)
    cols = [(int(j), mc.encoded[:, int(j)].copy(), bytes(mc.salts[int(j)]), merkle_path(mc.levels, dom, int(j))) for j in idx]
    return qv, prox, cols, ws, rs


def mask_verify(root: bytes, specs, functionals, opening, tr: "Transcript", tag: "HashTag" = None, log_msg: int = MASK_LOG_MSG,
                log_dom: int = MASK_LOG_DOM, q: int = MASK_Q) -> Optional[str]:
    """zk.rs:658-700 (mask_verify) / :712-760 (mask_verify_tagged): None when accepted, else the refusal's text."""
    tag = tag or HashTag.legacy()
    qv, prox, cols = opening[0], opening[1], opening[2]
    m, dom, S = 1 << log_msg, 1 << log_dom, len(specs)
    n_base = 2 * S + 4
    theta = tr.challenge_fp2()
    ws, v = mask_combined_weights(specs, functionals, theta, m)
    if len(qv) != 2 * m:
        return "mask: q length"
    got = fp2_mul_base(fp2_add(tuple(int(t) for t in qv[0]), tuple(int(t) for t in qv[m])), m)
    if got != v:
        return "mask: the product polynomial's sum != the combined functional"
    tr.absorb_fp2(b"mask-q", qv)
    rs = tr.challenge_fp2_vec(2 * S + 2)
    if len(prox) != 2 * m:
        return "mask: prox length"
    tr.absorb_fp2(b"mask-prox", prox)
    idx = tr.challenge_indices(q, dom)
    if len(cols) != len(idx):
        return "mask: column count"
    pows = coset_powers(7, dom)
    enc = lambda c: encode_coeffs_coset(c, pows, log_dom)
    w_enc = [(enc(ntt_inverse(ws[s, :, 0], log_dom)), enc(ntt_inverse(ws[s, :, 1], log_dom))) for s in range(S)]
    q_enc, p_enc = (enc(qv[:, 0]), enc(qv[:, 1])), (enc(prox[:, 0]), enc(prox[:, 1]))
    for (j, col, salt, path), want in zip(cols, idx):
        if j != int(want):
            return "mask: column index"
        if len(col) != n_base:
            return "mask: column length"
        leaf = salt_leaves(hash_columns(np.ascontiguousarray(col).reshape(n_base, 1), n_base, 1, tag.column), np.frombuffer(salt, np.uint8).reshape(1, 32), tag.leaf)
        if not merkle_verify_path(root, j, bytes(leaf[0]), path, tag.node):
            return f"mask: Merkle path for column {j} fails"
        acc = (int(col[2 * S]), int(col[2 * S + 1]))
        for s in range(S):
            acc = fp2_add(acc, fp2_mul((int(col[2 * s]), int(col[2 * s + 1])), (int(w_enc[s][0][j]), int(w_enc[s][1][j]))))
        if acc != (int(q_enc[0][j]), int(q_enc[1][j])):
            return f"mask: column {j} disagrees with the product polynomial"
        pacc = (int(col[n_base - 2]), int(col[n_base - 1]))
        for row in range(2 * S + 2):
            pacc = fp2_add(pacc, fp2_mul_base((int(rs[row, 0]), int(rs[row, 1])), int(col[row])))
        if pacc != (int(p_enc[0][j]), int(p_enc[1][j])):
            return f"mask: column {j} disagrees with the proximity vector"
    return None


# ----------------------------------------------------------------------------- witness weight products
def witness_product(t_rows: int, x, xs: int, w, inner: int, outer: int, os_: int, out_len: int, in_out: bool) -> np.ndarray:
    """witness.rs:979-991 (matmul_reference)"""
    x, w = np.ascontiguousarray(x, np.int64), np.ascontiguousarray(w, np.int8)
    assert (t_rows - 1) * xs + inner <= x.size and inner * outer <= w.size and (t_rows - 1) * os_ + outer <= out_len
    out = np.empty(out_len, dtype=np.int64)
    _lib.or_witness_product(C.c_size_t(t_rows), _p(x), C.c_size_t(xs), _p(w), C.c_size_t(inner), C.c_size_t(outer), C.c_size_t(os_),
                            C.c_size_t(out_len), C.c_int(1 if in_out else 0), _p(out))
    return out
