"""Regenerates the fixtures in this folder from the reference's own golden data.

Run once, in a checkout that has the reference tree mounted:

    python tests/golden/make_golden.py <path to the reference checkout>

It copies DATA only (recorded test vectors and agreement corpora), never source:

* ``encode_vectors.json`` - the 35 row-encoding digests, the definitional full rows and the
  named-bug digests of ``results/zk60_encode_vectors/{vectors,full_rows,negative_controls}.json``
  (the contract of ``zkp-core/src/pcs/encode_conformance_tests.rs``), reduced to the fields the
  tests read;
* ``l5_corpus.txt`` - ``results/zk60_lean_l5_20261106/corpus.txt`` (field, BLAKE3, transcript,
  Merkle and whole seeded tagged openings; grammar in ``zkp-core/tests/lean_l5_export.rs``);
* ``l6_corpus.txt`` - ``results/zk60_lean_l6_20261106/corpus.txt`` (eq tables, interpolation, CFS
  masks, whole sumchecks; grammar in ``zkp-core/tests/lean_l6_export.rs``).
"""
import json
import os
import shutil
import sys


def main(ref: str) -> None:
    here = os.path.dirname(os.path.abspath(__file__))
    ev = os.path.join(ref, "results", "zk60_encode_vectors")
    vec = json.load(open(os.path.join(ev, "vectors.json")))
    rows = json.load(open(os.path.join(ev, "full_rows.json")))["rows"]
    neg = json.load(open(os.path.join(ev, "negative_controls.json")))["entries"]
    keep = ("name", "log_n", "n", "inv_rate", "nn", "q_pad", "coset_h", "msg_seed", "pad_seed", "msg_sha256",
            "pad_sha256", "encoded_sha256", "encoded_first8", "encoded_last8", "encoded_probes")
    out = {
        "meta": {k: vec["meta"][k] for k in ("field_modulus", "two_adic_root_32", "coset_generator", "digest_rule", "prng")},
        "vectors": [{k: v[k] for k in keep} for v in vec["vectors"]],
        "full_rows": {k: r for k, r in rows.items() if k.startswith(("w3r4", "w4r4", "w6r4"))},
        "negative_controls": [
            {"vector": e["vector"], "correct_sha256": e["correct_sha256"],
             "controls": [{"bug": c["bug"], "sha256": c["sha256"]} for c in e["controls"]]}
            for e in neg
        ],
    }
    with open(os.path.join(here, "encode_vectors.json"), "w") as f:
        json.dump(out, f, separators=(",", ":"))
    shutil.copyfile(os.path.join(ref, "results", "zk60_lean_l5_20261106", "corpus.txt"), os.path.join(here, "l5_corpus.txt"))
    shutil.copyfile(os.path.join(ref, "results", "zk60_lean_l6_20261106", "corpus.txt"), os.path.join(here, "l6_corpus.txt"))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
