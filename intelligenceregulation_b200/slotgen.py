"""Generates one compiled sumcheck round kernel per known slot expression graph.

    python -m intelligenceregulation_b200.slotgen [out_dir]

The reference's Metal backend generates a kernel per slot from the slot's expression graph
(hashline/src/private_block/metal_slot.rs:115-497: `msl_round_kernels`, `lin_plan`, `gen_kernel`); this is the CUDA
counterpart.  Inputs: the graphs under slot_graphs/ (the 23 recorded graphs of the 125M shape, structure only, and the 23
graphs of a real W16R2 block core).  Output: csrc/gen/slot_gen_<k>.cu (straight-line evaluation code, csrc/slot_gen.cuh has
the run-time support) and csrc/gen/slot_gen_table.cu (the signature table).

A kernel is found at run time by the SIGNATURE of the program the caller hands to hl_b200_rounds_new_ir: the word stream of
include/hl_b200.h with every coefficient word replaced by the coefficient's class (one, minus one, zero, base-valued,
extension-valued), so that the same graph is recognised whatever its challenges are.  The generated code reads its
coefficients by occurrence (the j-th coefficient word of the stream).  Two typings are emitted per graph: the first round,
in which the tables the graph's source records as base-valued are read as base words (the dispatcher checks the actual
tables before it uses this variant), and the later rounds, in which every table is extension-valued.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, List, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
GRAPHS = os.path.join(HERE, "slot_graphs")
OUT = os.path.join(HERE, "csrc", "gen")
N_FILES = 8

ONE, NEG_ONE, ZERO, BASE, EXT = 0xFFFFFFFF, 0xFFFFFFFE, 0xFFFFFFFD, 0xFFFFFFF0, 0xFFFFFFF1
CLASS_WORD = {"one": ONE, "neg-one": NEG_ONE, "zero": ZERO, "base": BASE, "ext": EXT}
NODE_FLAG = 0x80000000
P = 0xFFFFFFFF00000001


class Graph:
    """tables: per table True when base-valued in the first round; nodes: ("affine", konst class, [(class, table)]) or
    ("sum", [(class, [factor])]); terms: [(class, [factor])]; a factor is ("t", id) or ("n", id).  Classes in stream order."""

    def __init__(self, name: str, base: List[bool]):
        self.name, self.base, self.nodes, self.terms = name, base, [], []

    def stream(self) -> List[int]:
        """the word stream of include/hl_b200.h with coefficient classes in place of coefficient indices"""
        w: List[int] = []

        def fac(f):
            return (NODE_FLAG | f[1]) if f[0] == "n" else f[1]

        for nd in self.nodes:
            if nd[0] == "affine":
                w += [0 | (len(nd[2]) << 8), CLASS_WORD[nd[1]]]
                for c, t in nd[2]:
                    w += [CLASS_WORD[c], t]
            else:
                w.append(1 | (len(nd[1]) << 8))
                for c, fs in nd[1]:
                    w += [CLASS_WORD[c], len(fs)] + [fac(f) for f in fs]
        for c, fs in self.terms:
            w += [CLASS_WORD[c], len(fs)] + [fac(f) for f in fs]
        return w

    def signature(self) -> int:
        h = 0xCBF29CE484222325
        for word in [len(self.base), len(self.nodes), len(self.terms)] + self.stream():
            for b in int(word).to_bytes(4, "little"):
                h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
        return h

    def n_coefs(self) -> int:
        n = 0
        for nd in self.nodes:
            n += 1 + len(nd[2]) if nd[0] == "affine" else len(nd[1])
        return n + len(self.terms)


def _m125_graphs() -> List[Graph]:
    out = []
    cls = {"one": "one", "kbase": "base", "chal": "ext"}
    for s in json.load(open(os.path.join(GRAPHS, "m125.json")))["slots"]:
        g = Graph("m125_" + s["name"], [f == "base" for f in s["table_fields"]])

        def fac(f):
            return ("n", f["n"]) if "n" in f else ("t", f["t"])

        for nd in s["nodes"]:
            if "affine" in nd:
                g.nodes.append(("affine", "base" if nd["konst"] else "zero", [(cls[c], t) for c, t in nd["affine"]]))
            else:
                g.nodes.append(("sum", [(cls[c], [fac(f) for f in fs]) for c, fs in nd["sum"]]))
        for t in s["terms"]:
            g.terms.append((cls[t["coef"]], [("t", x) for x in t["wrapper"]] + [fac(f) for f in t["inner"]]))
        out.append(g)
    return out


def _w16r2_graphs() -> List[Graph]:
    out = []

    def cls(c):  # by value, as the flattening of a `SlotIr` classifies its coefficients
        v = (c[0], c[1])
        return "one" if v == (1, 0) else "neg-one" if v == (P - 1, 0) else "zero" if v == (0, 0) else "base" if c[1] == 0 else "ext"

    for s in json.load(open(os.path.join(GRAPHS, "w16r2.json")))["slots"]:
        matmul = 5 <= s["slot"] <= 13
        base = [not (k in ("eq", "geq", "H") or (k == "pub" and matmul)) for k in s["tables"]]
        g = Graph("w16r2_slot%d" % s["slot"], base)
        for nd in s["nodes"]:
            if "affine" in nd:
                g.nodes.append(("affine", cls(nd["konst"]), [(cls(c), t) for c, t in nd["affine"]]))
            else:
                g.nodes.append(("sum", [(cls(c), [tuple(f) for f in fs]) for c, fs in nd["sum"]]))
        for t in s["terms"]:
            g.terms.append((cls(t["coef"]), [("t", x) for x in t["wrapper"]] + [tuple(f) for f in t["inner"]]))
        out.append(g)
    return out


def all_graphs() -> List[Graph]:
    seen: Dict[int, Graph] = {}
    for g in _w16r2_graphs() + _m125_graphs():
        seen.setdefault(g.signature(), g)
    return list(seen.values())


# ------------------------------------------------------------------------------------------------ code emission
class Emitter:
    """Straight-line code of one typing of one graph; a value is (is_ext, C expression).

    Nodes are emitted DEPTH FIRST from the terms: a node's code sits inside its first consumer's accumulation, right before
    the product that needs it, so that a value used once dies at once and the registers hold little more than the open
    accumulators of the current path through the graph (the stream's own order computes every node first and keeps all of
    them alive to the end, which the compiler answers with kilobytes of spills on the 60-table graphs)."""

    RELOAD_AFTER = 60  # a table value is kept for this many emitted lines after its last use, then read again (its words are in L1)

    def __init__(self, g: Graph, first_round: bool):
        self.g, self.r0 = g, first_round
        self.lines: List[str] = []
        self.tab: Dict[int, Tuple[bool, str]] = {}
        self.last_use: Dict[int, int] = {}
        self.loads = 0
        self.tmp = 0
        self.done: Dict[int, Tuple[bool, str]] = {}
        # coefficient occurrences in STREAM order, whatever order the code is emitted in
        self.occ: List[List[int]] = []
        k = 0
        for nd in g.nodes:
            cnt = 1 + len(nd[2]) if nd[0] == "affine" else len(nd[1])
            self.occ.append(list(range(k, k + cnt)))
            k += cnt
        self.term_occ = list(range(k, k + len(g.terms)))
        # static types, in stream order (a node refers back only)
        self.ntype: List[bool] = []
        for nd in g.nodes:
            prods = self.products(nd)
            self.ntype.append(any(self.product_type(c, fs) for c, fs in prods if c != "zero"))

    @staticmethod
    def products(nd):
        """a node as [(class, [factor])]; an affine node's constant is a product without factors"""
        if nd[0] == "affine":
            return [(nd[1], [])] + [(c, [("t", t)]) for c, t in nd[2]]
        return nd[1]

    def emit(self, s: str) -> None:
        self.lines.append("        " + s)

    def table_type(self, t: int) -> bool:
        return not (self.r0 and self.g.base[t])

    def peek_type(self, f) -> bool:
        return self.ntype[f[1]] if f[0] == "n" else self.table_type(f[1])

    def product_type(self, cls: str, facs) -> bool:
        return cls == "ext" or any(self.peek_type(f) for f in facs)

    def table(self, t: int) -> Tuple[bool, str]:
        if t not in self.tab or len(self.lines) - self.last_use[t] > self.RELOAD_AFTER:
            ext = self.table_type(t)
            self.loads += 1
            name = ("te%d_%d" if ext else "tb%d_%d") % (t, self.loads)
            self.emit("const %s %s = sg::%s(T + 2 * (size_t)%d * stride, i, half, p);" % ("fp2" if ext else "u64", name, "ld_e" if ext else "ld_b", t))
            self.tab[t] = (ext, name)
        self.last_use[t] = len(self.lines)
        return self.tab[t]

    def factor(self, f) -> Tuple[bool, str]:
        return self.node(f[1]) if f[0] == "n" else self.table(f[1])

    def coef_value(self, cls: str, k: int):
        if cls in ("one", "neg-one", "zero"):
            return None
        return (True, "cf[%d]" % k) if cls == "ext" else (False, "cf[%d].c0" % k)

    def fresh(self, ext: bool) -> str:
        self.tmp += 1
        return ("xe%d" if ext else "xb%d") % self.tmp

    def mul(self, a, b) -> Tuple[bool, str]:
        """a reduced product as a new temporary"""
        if a[0] and b[0]:
            e = "sg::mul_ee(%s, %s)" % (a[1], b[1])
        elif a[0] or b[0]:
            x, y = (a, b) if a[0] else (b, a)
            e = "sg::mul_eb(%s, %s)" % (x[1], y[1])
        else:
            e = "sg::mul_bb(%s, %s)" % (a[1], b[1])
        ext = a[0] or b[0]
        name = self.fresh(ext)
        self.emit("const %s %s = %s;" % ("fp2" if ext else "u64", name, e))
        return ext, name

    def accumulate(self, acc: str, acc_ext: bool, cls: str, cval, facs, constant_term: bool) -> bool:
        """acc += coefficient * product(factors); returns True when an extension x extension product went in"""
        if cls == "zero":
            return False
        if constant_term and cval is not None:  # an affine node's constant: added as it is
            if acc_ext:
                self.emit(("sg::add_e(%s, %s);" if cval[0] else "sg::add_b(%s, %s);") % (acc, cval[1]))
            else:
                self.emit("sg::addw(%s, %s);" % (acc, cval[1]))
            return False
        vals = [self.factor(f) for f in facs]  # emits the factor nodes that are not computed yet, and the table loads
        if cval is not None:
            vals.append(cval)
        vals = sorted(vals, key=lambda v: v[0])  # base factors first: their products are the cheap ones
        if not vals:  # a constant 1 or -1
            word = "1" if cls == "one" else "%dull" % (P - 1)
            self.emit(("sg::add_b(%s, %s);" if acc_ext else "sg::addw(%s, %s);") % (acc, word))
            return False
        if cls == "neg-one":
            v0 = vals[0]
            name = self.fresh(v0[0])
            self.emit("const %s %s = %s(%s);" % ("fp2" if v0[0] else "u64", name, "sg::neg_e" if v0[0] else "sg::neg_b", v0[1]))
            vals = [(v0[0], name)] + vals[1:]
        if len(vals) == 1:
            v = vals[0]
            if acc_ext:
                self.emit(("sg::add_e(%s, %s);" if v[0] else "sg::add_b(%s, %s);") % (acc, v[1]))
            else:
                self.emit("sg::addw(%s, %s);" % (acc, v[1]))
            return False
        chain = vals[0]
        for v in vals[1:-1]:
            chain = self.mul(chain, v)
        last = vals[-1]
        if not acc_ext:
            self.emit("sg::mac(%s, %s, %s);" % (acc, chain[1], last[1]))
            return False
        if chain[0] and last[0]:
            self.emit("sg::mac_ee(%s, %s, %s);" % (acc, chain[1], last[1]))
            return True
        if chain[0] or last[0]:
            x, y = (chain, last) if chain[0] else (last, chain)
            self.emit("sg::mac_eb(%s, %s, %s);" % (acc, x[1], y[1]))
        else:
            self.emit("sg::mac_bb(%s, %s, %s);" % (acc, chain[1], last[1]))
        return False

    def sum_of(self, name: str, products, occ: List[int], ext: bool, affine: bool) -> Tuple[bool, str]:
        # one accumulator per nesting depth and type, reused by every node that is evaluated at that depth
        self.depth = getattr(self, "depth", -1) + 1
        self.max_depth = max(getattr(self, "max_depth", 0), self.depth)
        acc = ("ae%d" if ext else "ab%d") % self.depth
        if not hasattr(self, "accs"):
            self.accs = set()
        self.accs.add(acc)
        self.emit(("%s = sg::acce_zero();" if ext else "%s = sg::acc_zero();") % acc)
        used7 = False
        for j, (c, fs) in enumerate(products):
            used7 |= self.accumulate(acc, ext, c, self.coef_value(c, occ[j]), fs, affine and j == 0)
        var = ("ne_%s" if ext else "nb_%s") % name
        if ext:
            self.emit("const fp2 %s = sg::red_e<%s>(%s);" % (var, "true" if used7 else "false", acc))
        else:
            self.emit("const u64 %s = sg::red(%s);" % (var, acc))
        self.emit("sg::fence();")
        self.depth -= 1
        return ext, var

    def node(self, j: int) -> Tuple[bool, str]:
        if j not in self.done:
            nd = self.g.nodes[j]
            self.done[j] = self.sum_of("n%d" % j, self.products(nd), self.occ[j], self.ntype[j], nd[0] == "affine")
        return self.done[j]

    def run(self) -> List[str]:
        ext = any(self.product_type(c, fs) for c, fs in self.g.terms if c != "zero")
        ext, var = self.sum_of("out", self.g.terms, self.term_occ, ext, False)
        self.emit("return %s;" % (var if ext else "f2(%s, 0)" % var))
        decl = []
        for kind, pre in (("sg::AccE", "ae"), ("sg::Acc", "ab")):
            names = sorted(a for a in self.accs if a.startswith(pre))
            if names:
                decl.append("        %s %s;" % (kind, ", ".join(names)))
        return decl + self.lines


def graph_code(g: Graph) -> str:
    sig = g.signature()
    has_r0 = any(g.base)
    mask = sum(1 << t for t, b in enumerate(g.base) if b)
    ext_body = Emitter(g, False).run()
    out = ["// %s: %d tables, %d nodes, %d terms, %d coefficient words" % (g.name, len(g.base), len(g.nodes), len(g.terms), g.n_coefs()),
           "struct G_%016x {" % sig,
           "    static constexpr u32 N_CFO = %d;" % g.n_coefs(),
           "    static constexpr bool HAS_R0 = %s;" % ("true" if has_r0 else "false"),
           "    template <bool R0>",
           "    static __device__ __forceinline__ fp2 eval(const u64* __restrict__ T, size_t stride, u32 i, u32 half, u32 p, const fp2* __restrict__ cf) {"]
    if has_r0:
        out += ["      if constexpr (R0) {"] + Emitter(g, True).run() + ["      } else {"] + ext_body + ["      }"]
    else:
        out += ext_body
    out += ["    }", "};",
            "static const sg::Entry E_%016x = {0x%016xull, %du, %du, 0x%xull, \"%s\", &sg::launch_graph<G_%016x>};" % (
                sig, sig, len(g.base), g.n_coefs(), mask, g.name, sig), ""]
    return "\n".join(out)


def generate(out_dir: str = OUT) -> List[str]:
    """writes the sources (only the ones whose text changed) and returns their file names"""
    os.makedirs(out_dir, exist_ok=True)
    graphs = sorted(all_graphs(), key=lambda g: -g.n_coefs())
    files: List[List[Graph]] = [[] for _ in range(N_FILES)]
    for j, g in enumerate(graphs):  # the largest graphs spread over the files, so that the files compile in similar time
        files[j % N_FILES].append(g)
    names = []

    def write(name: str, text: str) -> None:
        path = os.path.join(out_dir, name)
        if not os.path.exists(path) or open(path).read() != text:
            with open(path, "w") as f:
                f.write(text)
        names.append(name)

    head = "// GENERATED by slotgen.py from slot_graphs/*.json; do not edit.\n#include \"../slot_gen.cuh\"\n\nnamespace {\n\n"
    for k, gs in enumerate(files):
        body = head + "\n".join(graph_code(g) for g in gs) + "\n}  // namespace\n\n"
        body += "namespace sg {\nconst Entry* const* gen_entries_%d(int* n) {\n    static const Entry* const list[] = {%s};\n    *n = %d;\n    return list;\n}\n}  // namespace sg\n" % (
            k, ", ".join("&E_%016x" % g.signature() for g in gs) or "nullptr", len(gs))
        write("slot_gen_%d.cu" % k, body)
    table = "// GENERATED by slotgen.py; do not edit.\n#include \"../slot_gen.cuh\"\n\nnamespace sg {\n"
    table += "".join("const Entry* const* gen_entries_%d(int* n);\n" % k for k in range(N_FILES))
    table += "const Entry* find(u64 signature) {\n"
    for k in range(N_FILES):
        table += "    {\n        int n = 0;\n        const Entry* const* e = gen_entries_%d(&n);\n        for (int i = 0; i < n; i++)\n            if (e[i]->signature == signature) return e[i];\n    }\n" % k
    table += "    return nullptr;\n}\n}  // namespace sg\n"
    write("slot_gen_table.cu", table)
    return names


if __name__ == "__main__":
    for n in generate(sys.argv[1] if len(sys.argv) > 1 else OUT):
        print(n)
