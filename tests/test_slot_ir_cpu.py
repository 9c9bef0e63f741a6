"""Slot polynomials as data, without a device: the structural fixture of the reference's 23 slot graphs is
well formed, the oracle's interpreter (slot_ir.rs:352-377 restated in C) agrees with a pure-Python evaluation
and with the closed-form families, and the product's interpreter and program check, compiled for the host,
agree with the oracle.  Field work: bit-exact."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import ir_util as U

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def emul():
    src = os.path.join(ROOT, "tests", "host_emul", "slot_ir_emul.cpp")
    so = os.path.join(ROOT, "tests", "host_emul", "libslot_ir_emul.so")
    core = os.path.join(ROOT, "intelligenceregulation_b200", "csrc", "slot_ir.cuh")
    if not os.path.exists(so) or max(os.path.getmtime(src), os.path.getmtime(core)) > os.path.getmtime(so):
        subprocess.check_call(["/usr/bin/g++", "-std=c++17", "-O2", "-shared", "-fPIC", "-o", so, src])
    return C.CDLL(so)


def _vp(a):
    return C.c_void_p(a.ctypes.data)


def test_fixture_is_well_formed_and_degrees_match_the_reference(golden_dir):
    slots = U.load_slots(golden_dir)
    assert len(slots) == 23
    for s in slots:
        nd, td = U.degrees(s)
        for n, d in zip(s["nodes"], nd):
            if "sum" in n:
                assert d == n["degree"], (s["name"], n)
        assert td == [t["degree"] for t in s["terms"]], s["name"]
        # the attained degree never exceeds the declared one (slot_ir.rs:380-384)
        assert max(td) <= s["declared_degree"], s["name"]
    big = slots[14]
    assert len(big["table_fields"]) == 60 and len(big["nodes"]) == 71 and big["declared_degree"] == 5


def test_oracle_and_product_interpreters_agree_with_python_on_every_slot(oracle, emul, golden_dir):
    from intelligenceregulation_b200 import backend

    for s in U.load_slots(golden_dir):
        prog, desc = U.build_program(backend, s, 4000 + s["slot"])
        w, cf = prog.words(), prog.coef_array()
        k = prog.n_tables
        assert emul.emul_ir_validate(_vp(w), w.size, k, prog.n_nodes, prog.n_terms, cf.shape[0]) == 0, s["name"]
        oracle.ir_set(w, prog.n_nodes, prog.n_terms)
        rng = np.random.default_rng(s["slot"])
        for rep in range(3):
            v = rng.integers(0, U.P, size=(k, 2), dtype=np.uint64)
            want = U.py_eval(desc, [(int(a), int(b)) for a, b in v])
            assert oracle.poly_eval(oracle.POLY_IR, v, cf if cf.size else None) == want, (s["name"], rep)
            out = np.zeros(2, dtype=np.uint64)
            emul.emul_ir_eval(_vp(w), w.size, k, prog.n_nodes, prog.n_terms, _vp(cf) if cf.size else None, cf.shape[0], _vp(v), _vp(out))
            assert (int(out[0]), int(out[1])) == want, (s["name"], rep)
            # the evaluation plan the kernels run, walked by one worker (the thread form)
            info = np.zeros(5, dtype=np.uint32)
            out[:] = 0
            rc = emul.emul_ir_plan_eval(_vp(w), w.size, k, prog.n_nodes, prog.n_terms, _vp(cf) if cf.size else None, cf.shape[0], _vp(v),
                                        s["declared_degree"], _vp(out), _vp(info))
            assert rc == 0 and (int(out[0]), int(out[1])) == want, (s["name"], rep)
            assert info[1] == prog.n_nodes + 1
            assert info[4] == sum(1 for n in s["nodes"] if "affine" in n)


def test_pair_form_gives_the_values_at_every_point(oracle, emul, golden_dir):
    """the kernels' pair form (tables and affine nodes stepped by their differences, the other nodes level by level with
    one (unit, point) per lane) == the polynomial at T(i) + d (T(i+half) - T(i)), for 32 lanes and for 5, with and
    without the point 1"""
    from intelligenceregulation_b200 import backend

    for s in U.load_slots(golden_dir):
        prog, desc = U.build_program(backend, s, 5000 + s["slot"])
        w, cf = prog.words(), prog.coef_array()
        k, deg = prog.n_tables, s["declared_degree"]
        rng = np.random.default_rng(77 + s["slot"])
        lo = rng.integers(0, U.P, size=(k, 2), dtype=np.uint64)
        hi = rng.integers(0, U.P, size=(k, 2), dtype=np.uint64)
        de = min(deg, max(U.degrees(s)[1]))  # the kernels evaluate 0 .. min(declared, attained); the step extrapolates the rest
        want = []
        for d in range(deg + 1):
            v = [((int(a[0]) + d * (int(b[0]) - int(a[0]))) % U.P, (int(a[1]) + d * (int(b[1]) - int(a[1]))) % U.P) for a, b in zip(lo, hi)]
            want.append(U.py_eval(desc, v))
        for mode in (0, 1, 2):  # point by point; every point per unit; the same without the point 1
            out = np.zeros((deg + 1, 2), dtype=np.uint64)
            rc = emul.emul_ir_tpair(_vp(w), w.size, k, prog.n_nodes, prog.n_terms, _vp(cf) if cf.size else None, cf.shape[0], _vp(lo), _vp(hi),
                                    deg, mode, _vp(out))
            if rc == -1 and mode:
                continue  # beyond the all-points form's limits: the kernels use the point-by-point form there
            assert rc == 0
            exp = [(0, 0) if (mode == 2 and d == 1) else want[d] for d in range(de + 1)]
            assert [(int(a), int(b)) for a, b in out[: de + 1]] == exp, (s["name"], "thread pair form", mode)
        for lanes, skip in ((32, 0), (5, 1), (32, 1)):
            out = np.zeros((deg + 1, 2), dtype=np.uint64)
            rc = emul.emul_ir_pair(_vp(w), w.size, k, prog.n_nodes, prog.n_terms, _vp(cf) if cf.size else None, cf.shape[0], _vp(lo), _vp(hi),
                                   deg, lanes, skip, _vp(out))
            assert rc == 0
            for d in range(deg + 1):
                exp = (0, 0) if (skip and d == 1) or d > de else want[d]
                assert (int(out[d][0]), int(out[d][1])) == exp, (s["name"], d, lanes, skip)


def test_closed_form_families_written_as_programs(oracle):
    from intelligenceregulation_b200 import backend

    SP = backend.SlotProgram
    rng = np.random.default_rng(7)
    alpha = (int(rng.integers(0, U.P, dtype=np.uint64)), int(rng.integers(0, U.P, dtype=np.uint64)))
    fams = []
    p = SP(2); p.term(SP.ONE, [], [0, 1]); fams.append((oracle.POLY_PROD, p, None))
    p = SP(4); n = p.sum([(SP.ONE, [1, 2]), (SP.NEG_ONE, [3])]); p.term(SP.ONE, [0], [SP.node(n)]); fams.append((oracle.POLY_ZC, p, None))
    p = SP(3); a = p.affine(alpha, [(SP.NEG_ONE, 2)]); n = p.sum([(SP.ONE, [1, SP.node(a)]), (SP.NEG_ONE, [])]); p.term(SP.ONE, [0], [SP.node(n)])
    fams.append((oracle.POLY_LOGUP_Q, p, alpha))
    p = SP(4); a = p.affine(alpha, [(SP.NEG_ONE, 2)]); n = p.sum([(SP.ONE, [1, SP.node(a)]), (SP.NEG_ONE, [3])]); p.term(SP.ONE, [0], [SP.node(n)])
    fams.append((oracle.POLY_LOGUP_T, p, alpha))
    for fam, prog, al in fams:
        oracle.ir_set(prog.words(), prog.n_nodes, prog.n_terms)
        cf = prog.coef_array()
        for _ in range(4):
            v = rng.integers(0, U.P, size=(prog.n_tables, 2), dtype=np.uint64)
            want = oracle.poly_eval(fam, v, np.array(al, dtype=np.uint64) if al else None)
            assert oracle.poly_eval(oracle.POLY_IR, v, cf if cf.size else None) == want


def test_program_check_refuses_malformed_streams(emul, golden_dir):
    from intelligenceregulation_b200 import backend

    s = U.load_slots(golden_dir)[3]
    prog, _ = U.build_program(backend, s, 1)
    w, cf = prog.words(), prog.coef_array()
    k, nn, nt, nc = prog.n_tables, prog.n_nodes, prog.n_terms, cf.shape[0]

    def check(words, k=k, nn=nn, nt=nt, nc=nc):
        words = np.ascontiguousarray(words, dtype=np.uint32)
        return emul.emul_ir_validate(_vp(words), words.size, k, nn, nt, nc)

    assert check(w) == 0
    assert check(w[:-1]) != 0                      # truncated
    assert check(np.append(w, 0)) != 0             # trailing words
    assert check(w, k=k - 1) != 0                  # a table id out of range
    assert check(w, nc=max(nc - 1, 0)) != 0 or nc == 0   # a coefficient index out of range
    bad = w.copy()
    # first sum node: make one of its factors a forward node reference
    SP = backend.SlotProgram
    p2 = SP(2); p2.sum([(SP.ONE, [SP.node(0)])]); p2.term(SP.ONE, [0], [1])
    assert check(p2.words(), k=2, nn=1, nt=1, nc=0) != 0   # a node that refers to itself
    assert check(w, nn=nn + 1) != 0
    assert check(bad, k=65) != 0                   # beyond the table limit
