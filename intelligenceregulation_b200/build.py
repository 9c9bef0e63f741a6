"""Builds the backend's shared library in-tree with nvcc for sm_100a.

    python -m intelligenceregulation_b200.build [--force] [--verbose]

Output: ``intelligenceregulation_b200/libhl_b200.so`` (the C ABI of ``include/hl_b200.h``).
nvcc cross-compiles without a GPU; the library needs a B200 only when it is called.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libhl_b200.so")
SOURCES = ["api.cu", "commit_api.cu", "encode.cu", "hash.cu", "store.cu", "misc.cu", "sumcheck.cu", "rounds_api.cu", "hash_noalloc.cu", "logup.cu", "aux_api.cu", "tables.cu", "rng.cu", "lookup.cu", "mask.cu", "witness.cu", "act.cu", "verify.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the backend has no other build path")


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    graphs = os.path.join(HERE, "slot_graphs")
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f != "gen"] + [os.path.join(HERE, "..", "include", "hl_b200.h")]
    deps += [os.path.join(HERE, "slotgen.py")] + [os.path.join(graphs, f) for f in os.listdir(graphs)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    # the per-graph slot kernels are generated sources (csrc/gen/, not kept in the history)
    from . import slotgen

    gen_sources = [os.path.join("gen", f) for f in slotgen.generate()]
    objs = []
    obj_dir = os.path.join(HERE, "build")
    os.makedirs(obj_dir, exist_ok=True)
    common = [nvcc_path(), "-std=c++17", "-O3", "-lineinfo", "-ccbin", "/usr/bin/g++", "-Xcompiler", "-fPIC", "-Werror", "all-warnings", *ARCH]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    # a source is recompiled when it, or any header of the library, is newer than its object
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + [os.path.join(HERE, "..", "include", f) for f in ("hl_b200.h", "hl_b200_bench.h")]
    newest_header = max(os.path.getmtime(h) for h in headers)
    for src in SOURCES + gen_sources:
        obj = os.path.join(obj_dir, os.path.basename(src).replace(".cu", ".o"))
        objs.append(obj)
        if not force and not verbose and os.path.exists(obj) and os.path.getmtime(obj) > max(newest_header, os.path.getmtime(os.path.join(CSRC, src))):
            continue
        procs.append((src, subprocess.Popen(common + ["-c", os.path.join(CSRC, src), "-o", obj], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([nvcc_path(), "-shared", "-ccbin", "/usr/bin/g++", *ARCH, "-o", LIB, *objs, "-lcudart_static", "-lpthread", "-ldl", "-lrt"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
