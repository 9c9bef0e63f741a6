"""The reference's OWN CUDA kernels, compiled unchanged for sm_100a and launched with the reference's own launch shapes.

TEST AND BENCHMARK INFRASTRUCTURE, like everything under oracle/: the product never imports this file.  It serves two
purposes: a second, independent parity pin (the device results of this repository's kernels must equal what the reference's
kernels write, on the same inputs), and the performance bar "the reference's sm_100 kernel on the same GPU".

Source: hashline/src/gpu/kernels.cu of the reference tree (an NVRTC source file with no includes; the reference's
NVRTC arch table has a compute_100 arm, cuda.rs:561-577).  `build()` compiles it WHERE IT LIES into the git-ignored
oracle/_ref/kernels.cubin (`make -C oracle ref_cuda REF=<reference checkout>`); no source is copied.  Where the reference
tree is absent (the GPU box), the prebuilt cubin is used.

Launch shapes follow hashline/src/gpu/cuda.rs (cited at each method); `for_num_elems(n)` there is cudarc's
1,024-thread blocks over ceil(n / 1024) CTAs.  Every size is checked on the host before a launch: the kernels index with
32-bit ints and trust their arguments.

Device memory is torch tensors of int64 (the words are u64), launches go to torch's current stream.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional, Sequence, Tuple

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
CUBIN = os.path.join(HERE, "_ref", "kernels.cubin")
REF_SOURCE = "ops/zkp-mvp/gpu-metal/hashline/src/gpu/kernels.cu"
DEFAULT_REF = "/root/reference"
P = 0xFFFFFFFF00000001
NTT_LOG_BLK = 12          # cuda.rs:59
NTT_THREADS = 512         # cuda.rs:60-67 (the default of ntt_threads())


def build(ref_root: str = DEFAULT_REF, force: bool = False) -> Optional[str]:
    """Compiles the reference's kernels.cu for sm_100a when the reference tree is present; returns the cubin's path, or None
    when neither the tree nor a prebuilt cubin exists."""
    src = os.path.join(ref_root, REF_SOURCE)
    if os.path.exists(src) and (force or not os.path.exists(CUBIN) or os.path.getmtime(CUBIN) < os.path.getmtime(src)):
        subprocess.check_call(["make", "-C", HERE, "ref_cuda", f"REF={ref_root}"], stdout=subprocess.DEVNULL)
    return CUBIN if os.path.exists(CUBIN) else None


def available() -> bool:
    return os.path.exists(CUBIN)


def _fp_pow(a: int, e: int) -> int:
    return pow(a, e, P)


def two_adic_root(k: int) -> int:
    """field.rs:86-91: 7^((p-1)/2^32) raised to 2^(32-k)"""
    return _fp_pow(_fp_pow(7, (P - 1) >> 32), 1 << (32 - k))


def stage_major_twiddles(max_log: int) -> Tuple[np.ndarray, np.ndarray]:
    """cuda.rs:1624-1634 over ntt.rs:21-43: stage s (half = 2^(s-1)) owns entries [half - 1, 2 half - 1) = w_{2^s}^k, k < half;
    forward and inverse tables."""
    out = []
    for inverse in (False, True):
        t = np.empty((1 << max_log) - 1, dtype=np.uint64)
        for s in range(1, max_log + 1):
            half = 1 << (s - 1)
            w = two_adic_root(s)
            if inverse:
                w = _fp_pow(w, P - 2)
            cur = 1
            for k in range(half):
                t[half - 1 + k] = cur
                cur = cur * w % P
        out.append(t)
    return out[0], out[1]


class RefCuda:
    """The loaded module and one method per launch site of cuda.rs that this repository has a counterpart for."""

    KERNELS = ("k_ntt_p1", "k_ntt_p2_f", "k_zk_pad_scale", "k_dif_pa_f", "k_dif_pb", "k_dit_p1_pad_s", "k_hash_cols", "k_hash_cols_keyed",
               "k_fold_rows", "k_sc_fold", "k_eq_table", "k_eq_join", "k_helper", "k_widen", "k_gather_cols")

    def __init__(self, max_log: int = 16):
        import torch
        from cuda.bindings import driver as drv

        if not available():
            raise RuntimeError("oracle/_ref/kernels.cubin is not built (make -C oracle ref_cuda REF=<reference checkout>)")
        self.torch, self.drv = torch, drv
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # makes the primary context current on this thread
        err, self.mod = drv.cuModuleLoadData(open(CUBIN, "rb").read())
        self._ok(err, "cuModuleLoadData")
        self.fn = {}
        for name in self.KERNELS:
            err, f = drv.cuModuleGetFunction(self.mod, name.encode())
            self._ok(err, name)
            self.fn[name] = f
        self.max_log = max_log
        tf, ti = stage_major_twiddles(max_log)
        self.tw_f, self.tw_i = self.to_dev(tf), self.to_dev(ti)

    def _ok(self, err, what):
        if int(err) != 0:
            raise RuntimeError(f"reference CUDA harness: {what} failed with CUresult {int(err)}")

    def to_dev(self, a: np.ndarray):
        a = np.ascontiguousarray(a)
        if a.dtype == np.uint64:
            a = a.view(np.int64)
        return self.torch.from_numpy(a.copy()).cuda()

    def to_host_u64(self, t) -> np.ndarray:
        return t.cpu().numpy().view(np.uint64)

    def from_ptr(self, d_ptr: int, n_words: int):
        """a torch copy of `n_words` u64 at a raw device address (the owner's stream must be idle)"""
        out = self.torch.empty(n_words, dtype=self.torch.int64, device="cuda")
        self.torch.cuda.synchronize()
        (err,) = self.drv.cuMemcpyDtoD(out.data_ptr(), int(d_ptr), n_words * 8)
        self._ok(err, "cuMemcpyDtoD")
        return out

    def _launch(self, name: str, grid: Sequence[int], block: int, args: Sequence[Tuple[object, object]]) -> None:
        """args: (value, ctype) pairs; a torch tensor passes its device address"""
        gx, gy = (int(grid[0]), int(grid[1]) if len(grid) > 1 else 1)
        assert 1 <= gx < (1 << 31) and 1 <= gy < 65536 and 1 <= block <= 1024, (name, grid, block)
        vals, types = [], []
        for v, t in args:
            if t is C.c_void_p:
                v = int(v.data_ptr()) if hasattr(v, "data_ptr") else int(v)
            vals.append(v)
            types.append(t)
        stream = self.torch.cuda.current_stream().cuda_stream
        (err,) = self.drv.cuLaunchKernel(self.fn[name], gx, gy, 1, block, 1, 1, 0, stream, (tuple(vals), tuple(types)), 0)
        self._ok(err, name)

    @staticmethod
    def _for_num_elems(n: int) -> Tuple[Tuple[int], int]:
        return ((n + 1023) // 1024,), 1024

    # ------------------------------------------------------------------ transforms (cuda.rs:1678-1709 `ntt_rows`)
    def ntt_rows(self, src, dst, rows: int, n_src: int, log_n: int, inverse: bool) -> None:
        n = 1 << log_n
        assert 1 <= log_n <= self.max_log and log_n <= NTT_LOG_BLK + 12 and 1 <= n_src <= n and rows >= 1
        assert src.numel() >= rows * n_src and dst.numel() >= rows * n and rows * n < (1 << 31)
        tw = self.tw_i if inverse else self.tw_f
        scale = _fp_pow(n, P - 2) if inverse else 1
        lb = min(log_n, NTT_LOG_BLK)
        self._launch("k_ntt_p1", (rows << (log_n - lb),), NTT_THREADS,
                     [(src, C.c_void_p), (dst, C.c_void_p), (tw, C.c_void_p), (log_n, C.c_int), (n_src, C.c_int), (scale, C.c_uint64)])
        if log_n > NTT_LOG_BLK:
            self._launch("k_ntt_p2_f", (rows << (log_n - NTT_LOG_BLK),), NTT_THREADS,
                         [(dst, C.c_void_p), (tw, C.c_void_p), (log_n, C.c_int), (scale, C.c_uint64)])

    def encode_zk(self, data, pads, pows, rows: int, log_n: int, log_nn: int, q: int):
        """The resident hiding encode of cuda.rs:3731-3776 (`dev_commit_zk_from_inner`): inverse transform, pad + coset scale at
        width nn, forward transform of size nn.  Returns the rows x nn encoding."""
        n, nn = 1 << log_n, 1 << log_nn
        assert n + q <= nn and pads.numel() == rows * q and pows.numel() == nn and data.numel() == rows * n and rows * nn < (1 << 31)
        t = self.torch
        coef = t.empty(rows * n, dtype=t.int64, device="cuda")
        coef2 = t.empty(rows * nn, dtype=t.int64, device="cuda")
        enc = t.empty(rows * nn, dtype=t.int64, device="cuda")
        self.ntt_rows(data, coef, rows, n, log_n, True)
        grid, block = self._for_num_elems(rows * nn)
        self._launch("k_zk_pad_scale", grid, block, [(coef, C.c_void_p), (pads, C.c_void_p), (pows, C.c_void_p), (coef2, C.c_void_p),
                                                     (rows, C.c_int), (n, C.c_int), (q, C.c_int), (nn, C.c_int)])
        self.ntt_rows(coef2, enc, rows, nn, log_nn, False)
        return enc

    def encode_plain(self, data, rows: int, log_n: int, log_nn: int):
        """The systematic encode of cuda.rs:3578-3621 (`encode_rows`): DIF inverse (pass A strided, pass B contiguous, in place),
        then the padded DIT forward and its strided pass."""
        n, nn = 1 << log_n, 1 << log_nn
        assert log_nn <= self.max_log and log_n <= log_nn and data.numel() == rows * n and rows * nn < (1 << 31)
        t = self.torch
        coef = t.empty(rows * n, dtype=t.int64, device="cuda")
        enc = t.empty(rows * nn, dtype=t.int64, device="cuda")
        scale = _fp_pow(n, P - 2)
        if log_n > NTT_LOG_BLK:
            tiles = 1 << (log_n - NTT_LOG_BLK)
            self._launch("k_dif_pa_f", (rows * tiles,), NTT_THREADS, [(data, C.c_void_p), (coef, C.c_void_p), (self.tw_i, C.c_void_p), (log_n, C.c_int)])
            self._launch("k_dif_pb", (rows * tiles,), NTT_THREADS,
                         [(coef, C.c_void_p), (coef, C.c_void_p), (self.tw_i, C.c_void_p), (log_n, C.c_int), (scale, C.c_uint64)])
        else:
            self._launch("k_dif_pb", (rows,), NTT_THREADS,
                         [(data, C.c_void_p), (coef, C.c_void_p), (self.tw_i, C.c_void_p), (log_n, C.c_int), (scale, C.c_uint64)])
        rb, lb = log_nn - log_n, min(log_nn, NTT_LOG_BLK)
        self._launch("k_dit_p1_pad_s", (rows << (log_nn - lb),), NTT_THREADS,
                     [(coef, C.c_void_p), (enc, C.c_void_p), (self.tw_f, C.c_void_p), (log_nn, C.c_int), (n, C.c_int), (rb, C.c_int)])
        if log_nn > NTT_LOG_BLK:
            self._launch("k_ntt_p2_f", (rows << (log_nn - NTT_LOG_BLK),), NTT_THREADS,
                         [(enc, C.c_void_p), (self.tw_f, C.c_void_p), (log_nn, C.c_int), (1, C.c_uint64)])
        return enc

    # ------------------------------------------------------------------ column hash (cuda.rs:2928-2958)
    def hash_cols(self, enc, rows: int, nn: int, key: Optional[bytes]):
        assert enc.numel() >= rows * nn and rows >= 1 and nn >= 1 and rows * nn < (1 << 31) * 4
        t = self.torch
        leaves = t.empty(nn * 8, dtype=t.int32, device="cuda")
        grid, block = self._for_num_elems(nn)
        if key is None:
            self._launch("k_hash_cols", grid, block, [(enc, C.c_void_p), (leaves, C.c_void_p), (rows, C.c_int), (nn, C.c_int)])
        else:
            assert len(key) == 32
            dk = t.from_numpy(np.frombuffer(key, dtype="<u4").view(np.int32).copy()).cuda()  # cuda.rs:24-30 key_words
            self._launch("k_hash_cols_keyed", grid, block, [(enc, C.c_void_p), (leaves, C.c_void_p), (rows, C.c_int), (nn, C.c_int), (dk, C.c_void_p)])
            self.torch.cuda.current_stream().synchronize()  # the key words die with this frame
        return leaves

    # ------------------------------------------------------------------ opening fold (cuda.rs:3437-3460), at most 4 vectors
    def fold_rows(self, data, rhos, rows: int, n: int, k: int):
        assert 1 <= k <= 4 and data.numel() >= rows * n and rhos.numel() == k * rows * 2 and rows * n < (1 << 31)
        t = self.torch
        out = t.empty(k * n * 2, dtype=t.int64, device="cuda")
        grid, block = self._for_num_elems(n)
        self._launch("k_fold_rows", grid, block, [(data, C.c_void_p), (rhos, C.c_void_p), (out, C.c_void_p), (rows, C.c_int), (n, C.c_int), (k, C.c_int)])
        return out

    # ------------------------------------------------------------------ sumcheck fold (cuda.rs:3292-3293)
    def sc_fold(self, tabs, k: int, half: int, L: int, r: Tuple[int, int]) -> None:
        assert tabs.numel() >= k * L * 2 and 1 <= half and 2 * half <= L and k * L < (1 << 30)
        grid, block = self._for_num_elems(k * half)
        self._launch("k_sc_fold", grid, block, [(tabs, C.c_void_p), (k, C.c_int), (half, C.c_int), (L, C.c_int), (int(r[0]), C.c_uint64), (int(r[1]), C.c_uint64)])

    # ------------------------------------------------------------------ eq table (cuda.rs:3518-3541)
    def eq_table(self, r: np.ndarray):
        r = np.ascontiguousarray(r, dtype=np.uint64).reshape(-1, 2)
        nv = r.shape[0]
        assert 1 <= nv <= 26
        t = self.torch
        n = 1 << nv
        dst = t.empty(2 * n, dtype=t.int64, device="cuda")
        if nv <= 10:
            d_r = self.to_dev(r.reshape(-1))
            grid, block = self._for_num_elems(n)
            self._launch("k_eq_table", grid, block, [(d_r, C.c_void_p), (dst, C.c_void_p), (nv, C.c_int)])
            return dst
        lo_bits = nv // 2
        hi_bits = nv - lo_bits
        d_hi_r, d_lo_r = self.to_dev(r[:hi_bits].reshape(-1)), self.to_dev(r[hi_bits:].reshape(-1))
        d_hi = t.empty(2 << hi_bits, dtype=t.int64, device="cuda")
        d_lo = t.empty(2 << lo_bits, dtype=t.int64, device="cuda")
        grid, block = self._for_num_elems(1 << hi_bits)
        self._launch("k_eq_table", grid, block, [(d_hi_r, C.c_void_p), (d_hi, C.c_void_p), (hi_bits, C.c_int)])
        grid, block = self._for_num_elems(1 << lo_bits)
        self._launch("k_eq_table", grid, block, [(d_lo_r, C.c_void_p), (d_lo, C.c_void_p), (lo_bits, C.c_int)])
        grid, block = self._for_num_elems(n)
        self._launch("k_eq_join", grid, block, [(d_hi, C.c_void_p), (d_lo, C.c_void_p), (dst, C.c_void_p), (lo_bits, C.c_int), (n, C.c_int)])
        self.torch.cuda.current_stream().synchronize()  # the half tables die with this frame
        return dst

    # ------------------------------------------------------------------ LogUp helper column (cuda.rs:3478-3500)
    def helper(self, a, off_v1: int, off_w: int, off_v2: int, n: int, alpha, beta, c1, c2, h, off_re: int, off_im: int) -> None:
        """h = 1 / (alpha - (v1 + beta w + c1)) + 1 / (alpha - (v2 + c2)); off_w < 0: no w column"""
        assert n >= 1 and off_v1 >= 0 and off_v2 >= 0 and off_v1 + n <= a.numel() and off_v2 + n <= a.numel() and (off_w < 0 or off_w + n <= a.numel())
        assert off_re >= 0 and off_im >= 0 and off_re + n <= h.numel() and off_im + n <= h.numel() and a.numel() < (1 << 31) and h.numel() < (1 << 31)
        prm = self.to_dev(np.array([*alpha, *beta, *c1, *c2], dtype=np.uint64))
        threads = (n + 7) // 8
        self._launch("k_helper", ((threads + 127) // 128,), 128,
                     [(a, C.c_void_p), (off_v1, C.c_int), (off_w, C.c_int), (off_v2, C.c_int), (n, C.c_int), (prm, C.c_void_p), (h, C.c_void_p),
                      (off_re, C.c_int), (off_im, C.c_int)])
        self.torch.cuda.current_stream().synchronize()  # prm dies with this frame

    # ------------------------------------------------------------------ narrow witness planes (cuda.rs:1073-1105)
    def widen(self, src_bytes, n: int, w: int):
        assert w in (1, 2, 4) and src_bytes.numel() * src_bytes.element_size() >= n * w and n >= 1
        t = self.torch
        dst = t.empty(n, dtype=t.int64, device="cuda")
        grid, block = self._for_num_elems(n)
        self._launch("k_widen", grid, block, [(src_bytes, C.c_void_p), (dst, C.c_void_p), (n, C.c_longlong), (w, C.c_int)])
        return dst
