"""Writes the known slot expression graphs from the reference's own exports (data only; run where the reference is mounted):

    python intelligenceregulation_b200/slot_graphs/make_slot_graphs.py <path to the reference checkout>

The build generates one compiled round kernel per graph listed here (slotgen.py); bench.py replays the same graphs.

* m125.json           - the STRUCTURE of the 23 slot polynomials at the reference's recorded 125M shape
                        (results/zk60_slot_ir/slot_ir_m125.json; grammar private_block/slot_ir.rs:57-345): per slot its name,
                        round counts, declared degree, per table its field kind, per node and term the ids and coefficient classes.
* w16r2.json          - the 23 slot polynomials of a real W16R2 block core WITH their coefficient values and table kinds
                        (results/zk60_lean_l11_20261107/corpus.txt, records SLOT / IR / IRTAB / NODE / TERM; grammar
                        private_block/lean_l11_export_tests.rs:60-105).  The W16R2 profile is the one the Llama-3-8B block shape
                        (W16R2_8B_T128_H24) registers, so these graphs at that shape's cube sizes model a block's sumchecks.
"""
import json
import os
import sys


def fac(f):
    return {"n": f["node"]} if "node" in f else {"t": f["table"]}


def m125(ref_root, here):
    src = json.load(open(os.path.join(ref_root, "results", "zk60_slot_ir", "slot_ir_m125.json")))
    out = {"source": "results/zk60_slot_ir/slot_ir_m125.json", "shape": src["shape"], "slots": []}
    for s in src["slots"]:
        nodes = []
        for n in s["nodes"]:
            if n["kind"] == "affine":
                nodes.append({"affine": [[c["provenance"], c["table"]] for c in n["coefs"]], "konst": bool(n["has_const"])})
            else:
                nodes.append({"sum": [[st["coef_provenance"], [fac(f) for f in st["factors"]]] for st in n["subterms"]], "degree": n["degree"]})
        terms = [{"coef": t["coef_provenance"], "wrapper": t["wrapper"], "inner": [fac(f) for f in t["factors"]], "degree": t["degree"]} for t in s["terms"]]
        out["slots"].append({"slot": s["slot"], "name": s["name"], "main_rounds": s["main_rounds"], "extension_rounds": s["extension_rounds"],
                             "declared_degree": s["declared_degree"], "table_fields": [t["field"] for t in s["tables"]], "nodes": nodes, "terms": terms})
    json.dump(out, open(os.path.join(here, "m125.json"), "w"), separators=(",", ":"))


def l11(ref_root, here):
    def coef(c):
        c0, c1, cls = c.split(":")[:3]
        return [int(c0), int(c1), cls]

    def factors(s):
        return [] if s == "-" else [[f[0], int(f[1:])] for f in s.split(".")]

    slots, cur = [], None
    for line in open(os.path.join(ref_root, "results", "zk60_lean_l11_20261107", "corpus.txt")):
        w = line.rstrip("\n").split(" ")
        if w[0] == "SLOT":
            cur = {"slot": int(w[1]), "kind": w[2], "rung_rounds": int(w[3]), "ext": int(w[4]), "degree": int(w[5]), "tables": [], "nodes": [], "terms": []}
            slots.append(cur)
        elif w[0] == "IRTAB":
            cur["tables"].append(w[2].split(":")[0])
        elif w[0] == "NODE" and w[2] == "A":
            terms = [] if w[4] == "-" else [[coef(x.rsplit("@", 1)[0]), int(x.rsplit("@", 1)[1][1:])] for x in w[4].split(";")]
            cur["nodes"].append({"affine": terms, "konst": coef(w[3])})
        elif w[0] == "NODE":
            subs = [] if w[3] == "-" else [[coef(x.rsplit("@", 1)[0]), factors(x.rsplit("@", 1)[1])] for x in w[3].split(";")]
            cur["nodes"].append({"sum": subs})
        elif w[0] == "TERM":
            cur["terms"].append({"coef": coef(w[1]), "wrapper": [] if w[2] == "-" else [int(x) for x in w[2].split(",")], "inner": factors(w[3])})
    out = {"source": "results/zk60_lean_l11_20261107/corpus.txt", "profile": "W16R2_RUNG_H24", "slots": slots}
    json.dump(out, open(os.path.join(here, "w16r2.json"), "w"), separators=(",", ":"))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    here = os.path.dirname(os.path.abspath(__file__))
    m125(sys.argv[1], here)
    l11(sys.argv[1], here)
    for f in ("m125.json", "w16r2.json"):
        print(f, os.path.getsize(os.path.join(here, f)), "bytes")
