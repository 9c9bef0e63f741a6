"""Writes tests/golden/l11_corpus.txt from the reference's L11 agreement corpus
    results/zk60_lean_l11_20261107/corpus.txt
(written by hashline/src/private_block/lean_l11_export_tests.rs:102-262 from a REAL W16R2 block core: for each of the
23 slots the definition's draws, the proof's scalar, hosted terms, every round message, the terminal values, the table
list with eq points and small public tables, the slot's expression graph WITH its coefficient values, and the
verifier's recomputation `c, claimed, fin, rho, poly(vals), g` with the transcript state before and after).

Data only.  Prose is dropped: NLABEL lines go, IRTAB lines keep id and kind, a coefficient keeps `c0:c1:class` with
class one of one / neg-one / kbase / chal (the text after the class names the challenge in words).

Run in the build container (the reference tree is not present where the GPU tests run):
    python tests/golden/make_l11_golden.py <path to the reference checkout>
"""
import os
import sys


def coef(c: str) -> str:
    c0, c1, cls = c.split(":")[:3]
    return f"{c0}:{c1}:{cls}"


def prod(s: str) -> str:
    """`coef@factors` with the coefficient reduced to value and class"""
    c, f = s.rsplit("@", 1)
    return coef(c) + "@" + f


def main(ref_root: str) -> None:
    src = os.path.join(ref_root, "results", "zk60_lean_l11_20261107", "corpus.txt")
    out = []
    for line in open(src):
        w = line.rstrip("\n").split(" ")
        if w[0] == "NLABEL":
            continue
        if w[0] == "IRTAB":
            w = w[:3]
        elif w[0] == "NODE" and w[2] == "A":
            w = w[:3] + [coef(w[3]), "-" if w[4] == "-" else ";".join(prod(x) for x in w[4].split(";"))]
        elif w[0] == "NODE" and w[2] == "S":
            w = w[:3] + ["-" if w[3] == "-" else ";".join(prod(x) for x in w[3].split(";"))]
        elif w[0] == "TERM":
            w = [w[0], coef(w[1])] + w[2:]
        out.append(" ".join(w))
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "l11_corpus.txt")
    with open(dst, "w") as f:
        f.write("\n".join(out) + "\n")
    print(dst, os.path.getsize(dst), "bytes,", len(out), "records")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
