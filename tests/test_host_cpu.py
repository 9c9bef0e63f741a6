"""CPU-side checks: the C-ABI library loads and exports what the header declares, the kernels'
index arithmetic (run thread by thread on the host) reproduces the oracle's rows, and the
backend refuses to work without a device instead of falling back."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from intelligenceregulation_b200 import _lib, build

    build.build()
    lib = _lib.load()
    hdr = open(os.path.join(ROOT, "include", "hl_b200.h")).read() + open(os.path.join(ROOT, "include", "hl_b200_bench.h")).read()
    declared = set(re.findall(r"\b(hl_b200_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/hl_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


def test_no_device_means_an_error_not_a_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from intelligenceregulation_b200 import backend

    with pytest.raises(backend.DeviceError):
        backend.Context(0)


def test_misaligned_device_pointers_are_refused_before_any_cuda_call():
    """The allocation-free column hash loads words as u64 and stores leaves as u32: a pointer that is not aligned for that
    is a bad argument, answered on the host (no device is needed to be told so)."""
    from intelligenceregulation_b200 import _lib

    lib = _lib.load()
    ok_enc, ok_out = 0x10000, 0x20000  # never dereferenced: the refusal comes first
    assert lib.hl_b200_hash_columns_static(C.c_void_p(ok_enc + 4), 130, 1024, None, C.c_void_p(ok_out), None) == -1
    assert lib.hl_b200_hash_columns_static(C.c_void_p(ok_enc), 130, 1024, None, C.c_void_p(ok_out + 2), None) == -1


def test_product_does_not_reach_the_oracle():
    pkg = os.path.join(ROOT, "intelligenceregulation_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "hl_oracle" not in text and "oracle/" not in text, f"{f} names the oracle"


@pytest.fixture(scope="module")
def emul():
    src = os.path.join(ROOT, "tests", "host_emul", "encode_emul.cpp")
    so = os.path.join(ROOT, "tests", "host_emul", "libencode_emul.so")
    core = os.path.join(ROOT, "intelligenceregulation_b200", "csrc", "encode_core.cuh")
    if not os.path.exists(so) or max(os.path.getmtime(src), os.path.getmtime(core)) > os.path.getmtime(so):
        subprocess.check_call(["/usr/bin/g++", "-std=c++17", "-O2", "-shared", "-fPIC", "-o", so, src])
    return C.CDLL(so)


CASES = [  # fast, log_n, inv_rate, rows, q, zk, emulated threads
    (0, 3, 4, 2, 4, 1, 7), (0, 3, 4, 2, 12, 1, 32), (0, 6, 8, 3, 8, 1, 32), (0, 4, 4, 3, 0, 0, 5), (0, 1, 4, 2, 2, 1, 32),
    (1, 8, 2, 2, 8, 1, 32), (1, 8, 4, 2, 300, 1, 16), (1, 9, 4, 1, 8, 1, 32), (1, 10, 4, 2, 256, 1, 64), (1, 11, 2, 1, 40, 1, 128),
    (1, 12, 4, 1, 8, 0, 256), (1, 13, 2, 1, 280, 1, 512), (1, 14, 2, 1, 280, 1, 512), (1, 10, 4, 2, 0, 0, 64),
    # rows longer than one shared-memory transform (the T256 / T512 profiles, shape.rs:248-262): 2 and 4 residues each way
    (1, 15, 2, 1, 280, 1, 512), (1, 16, 2, 1, 280, 1, 512), (1, 15, 4, 1, 0, 0, 512), (1, 15, 4, 1, 40000, 1, 512),
]


@pytest.mark.parametrize("case", CASES)
def test_encoder_phases_on_the_host_match_the_oracle(emul, oracle, case):
    fast, logn, R, rows, q, zk, nt = case
    n, nn, logr = 1 << logn, (1 << logn) * R, R.bit_length() - 1
    rng = np.random.default_rng(1000 + logn * 16 + R)
    data = rng.integers(0, oracle.P, size=rows * n, dtype=np.uint64)
    pads = rng.integers(0, oracle.P, size=rows * max(q, 1), dtype=np.uint64)
    pows = oracle.coset_powers(7, nn)
    out = np.zeros(rows * nn, dtype=np.uint64)
    rc = emul.emul_encode(fast, C.c_void_p(data.ctypes.data), rows, logn, logr, C.c_void_p(pads.ctypes.data), q,
                          C.c_void_p(pows.ctypes.data), zk, nt, C.c_void_p(out.ctypes.data))
    assert rc == 0
    want = oracle.encode_rows_zk(data, rows, n, pads, q, pows, 18) if zk else oracle.encode_rows_plain(data, rows, n, nn, 18)
    assert (out == want).all()
