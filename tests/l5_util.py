"""The whole seeded openings of tests/golden/l5_corpus.txt as verifier inputs (exporter: zkp-core/tests/lean_l5_export.rs:342-427).
Each case rebuilds the exporter's data, claims and transcript start, and takes the OPENING from the records (`PCSG`, `PCSP`,
`PCSC`), so a verifier under test is handed what the reference's prover wrote and the reference's verifier accepted.  `MK` records are
single columns, honest and tampered, with the reference's own verdict on each."""
import numpy as np

CASES = {"rungg": ("hashline-zk-mr1/private-block-rung-g-t24-dev/1", 4, 4, 12, 31), "m125": ("hashline-zk-mr1/private-block-m125/1", 5, 2, 20, 32),
         "legacy": (None, 4, 4, 12, 33)}


def _fpv(s):
    return np.array([int(x) for x in s.split(",")], dtype=np.uint64) if s not in ("-", "") else np.zeros(0, dtype=np.uint64)


def _paths(s):
    return [bytes.fromhex(x) for x in s.split(",")] if s not in ("-", "") else []


def pcs_cases(o, l5):
    """[{name, tag, params, q, rows, claims, root, domain, opening, end_state, max_log}]"""
    out = []
    it = iter(l5)
    for r in it:
        if r[0] != "PCS":
            continue
        name = r[1]
        profile, log_cols, inv_rate, q, seed = CASES[name]
        tag = o.HashTag.for_profile(profile) if profile else o.HashTag.legacy()
        p = o.PcsParams(log_cols, inv_rate, q)
        n, rows = p.cols, 3
        rng = o.ZkRng(seed, b"lean-l5 pcs corpus")
        d = np.array([o.fp_from_i64(((i * 37) % 256) - 128) for i in range(rows * n)], dtype=np.uint64)
        for rr in (1, 2):
            for j in range(n):
                d[rr * n + j] = rng.fp()
        pt = np.array([[3000 + i * 7 + 3, 3 + i * 11 + 5] for i in range(log_cols)], dtype=np.uint64)
        e = (99991, 7)
        vp, vr = o.eval_mle_base(d[0:n], pt), o.eval_mle_base(d[n:2 * n], pt)
        one_e = o.fp2_sub((1, 0), e)
        claims = [o.ZClaim([o.ZPart(0, log_cols, one_e, pt), o.ZPart(n, log_cols, e, pt)], o.fp2_add(o.fp2_mul(one_e, vp), o.fp2_mul(e, vr)))]
        ng = int(r[7])
        gv = []
        for _ in range(ng):
            rec = next(it)
            assert rec[0] == "PCSG"
            gv.append(_fpv(rec[1]).reshape(-1, 2))
        rec = next(it)
        assert rec[0] == "PCSP"
        prox = _fpv(rec[1]).reshape(-1, 2)
        cols = []
        rec = next(it)
        while rec[0] == "PCSC":
            cols.append((int(rec[1]), _fpv(rec[2]), bytes.fromhex(rec[3]), _paths(rec[4])))
            rec = next(it)
        assert rec[0] == "PCSEND"
        out.append(dict(name=name, tag=tag, params=p, q=q, rows=rows, claims=claims, root=bytes.fromhex(r[3]), domain=bytes.fromhex(r[2]),
                        opening=o.OpeningZk(np.array(gv, dtype=np.uint64), prox, cols), end_state=bytes.fromhex(rec[1]), max_log=log_cols + 4))
    assert len(out) == 3
    return out


def start_transcript(o, case):
    tr = o.Transcript(case["domain"], case["tag"].transcript)
    tr.absorb(b"root", case["root"])
    return tr


def column_records(l5):
    """[(name, depth, rows, root, j, col, salt, path, verdict)] of the `MK` records"""
    out = []
    for r in l5:
        if r[0] == "MK":
            out.append((r[1], int(r[2]), int(r[3]), bytes.fromhex(r[4]), int(r[5]), _fpv(r[6]), bytes.fromhex(r[7]), _paths(r[8]), int(r[9])))
    assert len(out) == 84
    return out
