"""Shared by the slot-polynomial tests: the structural fixture of the reference's 23 slot graphs, a builder that
turns one into a `SlotProgram` with seeded coefficients, and an independent pure-Python evaluation."""
import json
import os

import numpy as np

P = 0xFFFFFFFF00000001


def load_slots(golden_dir):
    return json.load(open(os.path.join(golden_dir, "slot_ir_m125.json")))["slots"]


def f2_add(a, b):
    return ((a[0] + b[0]) % P, (a[1] + b[1]) % P)


def f2_mul(a, b):  # u^2 = 7 (field.rs:163-169)
    return ((a[0] * b[0] + 7 * a[1] * b[1]) % P, (a[0] * b[1] + a[1] * b[0]) % P)


class Rand:
    def __init__(self, seed):
        self.rng = np.random.default_rng(seed)

    def fp(self):
        return int(self.rng.integers(0, P, dtype=np.uint64))

    def coef(self, cls):
        if cls == "one":
            return "one"
        if cls == "kbase":  # a public base-field constant: small signed integers and powers of 256 in the reference
            v = int(self.rng.integers(-(1 << 40), 1 << 40))
            return (v % P, 0)
        return (self.fp(), self.fp())  # a challenge


def build_program(backend, slot, seed):
    """(SlotProgram, python-side description with concrete coefficient values) for one fixture slot"""
    SP = backend.SlotProgram
    r = Rand(seed)
    prog = SP(len(slot["table_fields"]))
    desc = {"nodes": [], "terms": []}

    def fw(f):
        return SP.node(f["n"]) if "n" in f else f["t"]

    for n in slot["nodes"]:
        if "affine" in n:
            konst = r.coef("kbase") if n["konst"] else "zero"
            terms = [(r.coef(c), t) for c, t in n["affine"]]
            prog.affine(konst, terms)
            desc["nodes"].append(("affine", konst, terms))
        else:
            subs = [(r.coef(c), [fw(f) for f in fs]) for c, fs in n["sum"]]
            prog.sum(subs)
            desc["nodes"].append(("sum", subs))
    for t in slot["terms"]:
        c = r.coef(t["coef"])
        prog.term(c, t["wrapper"], [fw(f) for f in t["inner"]])
        desc["terms"].append((c, list(t["wrapper"]) + [fw(f) for f in t["inner"]]))
    return prog, desc


def _cv(c):
    return {"one": (1, 0), "neg-one": (P - 1, 0), "zero": (0, 0)}[c] if isinstance(c, str) else c


def py_eval(desc, v):
    """private_block/slot_ir.rs:352-377 over Python integers; `v` = list of (c0, c1)"""
    nv = []

    def fv(f):
        return nv[f & 0x7FFFFFFF] if f & 0x80000000 else v[f]

    def prod(c, fs):
        p = _cv(c)
        for f in fs:
            p = f2_mul(p, fv(f))
        return p

    for n in desc["nodes"]:
        if n[0] == "affine":
            a = _cv(n[1])
            for c, t in n[2]:
                a = f2_add(a, f2_mul(_cv(c), v[t]))
        else:
            a = (0, 0)
            for c, fs in n[1]:
                a = f2_add(a, prod(c, fs))
        nv.append(a)
    tot = (0, 0)
    for c, fs in desc["terms"]:
        tot = f2_add(tot, prod(c, fs))
    return tot


def degrees(slot):
    """node and term degrees recomputed from the bodies (slot_ir.rs:386-413)"""
    d = []
    for n in slot["nodes"]:
        if "affine" in n:
            d.append(1 if n["affine"] else 0)
        else:
            d.append(max((sum(d[f["n"]] if "n" in f else 1 for f in fs) for _, fs in n["sum"]), default=0))
    td = [len(t["wrapper"]) + sum(d[f["n"]] if "n" in f else 1 for f in t["inner"]) for t in slot["terms"]]
    return d, td


def random_tables(slot, n_vars, seed):
    """(k, 2^n_vars, 2): base-field tables keep a zero imaginary word, as the reference's do (slot_ir.rs:160-177)"""
    rng = np.random.default_rng(seed)
    k = len(slot["table_fields"])
    t = rng.integers(0, P, size=(k, 1 << n_vars, 2), dtype=np.uint64)
    for i, f in enumerate(slot["table_fields"]):
        if f == "base":
            t[i, :, 1] = 0
    return t
