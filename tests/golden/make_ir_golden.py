"""Writes tests/golden/slot_ir_m125.json: the STRUCTURE of the 23 slot polynomials at the reference's
recorded 125M shape, copied from the reference's own export
    results/zk60_slot_ir/slot_ir_m125.json        (written by results/zk60_slot_ir/slot_ir_inventory.py
                                                   from private_block/argument.rs; grammar: slot_ir.rs:57-345)
Data only: per slot its name, round counts, declared degree, per table its field kind, per node and term the
table / node ids and the class of every coefficient ("one", "kbase" = public base-field constant, "chal" =
challenge, i.e. an extension element).  Labels, notes and prose are dropped; coefficient VALUES are not in
the export (they are challenges), so the tests draw them from a seed by class.

Run in the build container (the reference tree is not present where the GPU tests run):
    python tests/golden/make_ir_golden.py <path to the reference checkout>
"""
import json
import os
import sys


def fac(f):
    return {"n": f["node"]} if "node" in f else {"t": f["table"]}


def main(ref_root: str) -> None:
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
                             "declared_degree": s["declared_degree"], "table_fields": [t["field"] for t in s["tables"]],
                             "nodes": nodes, "terms": terms})
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "slot_ir_m125.json")
    with open(dst, "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print(dst, os.path.getsize(dst), "bytes,", len(out["slots"]), "slots")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
