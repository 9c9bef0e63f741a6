"""Pins the CPU oracle against the reference's own golden data (no GPU needed).

Sources of the fixtures: ``tests/golden/make_golden.py``.  Record grammars:
``zkp-core/tests/lean_l5_export.rs`` and ``lean_l6_export.rs`` of the reference;
encode vectors: ``zkp-core/src/pcs/encode_conformance_tests.rs``.
"""
import hashlib
import json
import os

import numpy as np
import pytest

P = 0xFFFFFFFF00000001
M64 = (1 << 64) - 1


def _records(path):
    with open(path) as f:
        for line in f:
            if line.startswith("#") or not line.strip():
                continue
            yield line.rstrip("\n").split(" ")


@pytest.fixture(scope="module")
def l5(golden_dir):
    return list(_records(os.path.join(golden_dir, "l5_corpus.txt")))


@pytest.fixture(scope="module")
def l6(golden_dir):
    return list(_records(os.path.join(golden_dir, "l6_corpus.txt")))


def unhex(s):
    return b"" if s == "-" else bytes.fromhex(s)


def gen_bytes(seed, n):
    """`gen:<seed>:<len>` of lean_l5_export.rs:51-53."""
    i = np.arange(n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        v = i * np.uint64(0x9E3779B97F4A7C15) + np.uint64((seed * 0xD1B54A32D192ED03) & M64)
    return (v >> np.uint64(56)).astype(np.uint8).tobytes()


def gen_fp2(n):
    """`fgen:<n>` of lean_l5_export.rs:56-58 (Fp::new of each word)."""
    i = np.arange(n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        a = i * np.uint64(0x9E3779B97F4A7C15)
    a = np.where(a >= np.uint64(P), a - np.uint64(P), a)
    b = i ^ np.uint64(0xDEADBEEF)
    return np.stack([a, b], axis=1).astype(np.uint64)


def data_spec(s):
    if s.startswith("gen:"):
        _, seed, n = s.split(":")
        return gen_bytes(int(seed), int(n))
    if s.startswith("h:"):
        return bytes.fromhex(s[2:])
    raise ValueError(s)


def fp2v(s):
    if s == "-":
        return np.zeros((0, 2), dtype=np.uint64)
    return np.array([int(x) for x in s.split(",")], dtype=np.uint64).reshape(-1, 2)


def fpv(s):
    if s == "-":
        return np.zeros(0, dtype=np.uint64)
    return np.array([int(x) for x in s.split(",")], dtype=np.uint64)


def f2(s):
    a, b = s.split(",")
    return (int(a), int(b))


# --------------------------------------------------------------------------- L5: field
def test_l5_field_records(oracle, l5):
    o, n = oracle, 0
    for r in l5:
        if r[0] == "FP":
            op, a = r[1], [int(x) for x in r[2:]]
            got = {
                "add": lambda: o.fp_add(a[0], a[1]), "sub": lambda: o.fp_sub(a[0], a[1]), "mul": lambda: o.fp_mul(a[0], a[1]),
                "neg": lambda: o.fp_neg(a[0]), "inv": lambda: o.fp_inv(a[0]), "pow": lambda: o.fp_pow(a[0], a[1]),
                "new": lambda: o.fp_new(a[0]), "u128": lambda: o.fp_from_u128((a[0] << 64) | a[1]),
            }[op]()
            assert got == a[-1], r
            n += 1
        elif r[0] == "F2":
            op, a = r[1], [int(x) for x in r[2:]]
            if op == "add": got, want = o.fp2_add(a[0:2], a[2:4]), a[4:6]
            elif op == "sub": got, want = o.fp2_sub(a[0:2], a[2:4]), a[4:6]
            elif op == "mul": got, want = o.fp2_mul(a[0:2], a[2:4]), a[4:6]
            elif op == "neg": got, want = o.fp2_neg(a[0:2]), a[2:4]
            elif op == "mulbase": got, want = o.fp2_mul_base(a[0:2], a[2]), a[3:5]
            elif op == "inv": got, want = o.fp2_inv(a[0:2]), a[2:4]
            else: raise AssertionError(op)
            assert list(got) == want, r
            n += 1
        elif r[0] == "BY":
            if r[1] == "fp":
                assert int(r[2]).to_bytes(8, "little").hex() == r[3]
            elif r[1] == "fp2":
                assert (int(r[2]).to_bytes(8, "little") + int(r[3]).to_bytes(8, "little")).hex() == r[4]
            elif r[1] == "fp2from":
                b = bytes.fromhex(r[2])
                assert o.fp_new(int.from_bytes(b[:8], "little")) == int(r[3]) and o.fp_new(int.from_bytes(b[8:], "little")) == int(r[4])
            n += 1
    assert n > 4000
    assert o.two_adic_root(32) == 1753635133440165772  # field.rs:339


# --------------------------------------------------------------------------- L5: BLAKE3
def test_l5_blake3_records_and_python_module(oracle, l5):
    n = 0
    for r in l5:
        if r[0] != "B3":
            continue
        data = data_spec(r[3])
        if r[1] == "hash":
            got = oracle.blake3(data)
        elif r[1] == "keyed":
            got = oracle.blake3(data, bytes.fromhex(r[2]))
        else:
            got = oracle.derive_key(bytes.fromhex(r[2]), data)
        assert got.hex() == r[4], r[:4]
        n += 1
    assert n == 119
    # a second, independent check where the `blake3` wheel is importable (XOF lengths included)
    b3 = pytest.importorskip("blake3")
    key = bytes(range(32))
    for ln in (0, 1, 63, 64, 65, 1023, 1024, 1025, 2048, 3073, 7000, 20032, 32768):
        d = gen_bytes(ln + 3, ln)
        assert oracle.blake3(d) == b3.blake3(d).digest()
        assert oracle.blake3(d, key) == b3.blake3(d, key=key).digest()
        assert oracle.blake3(d, None, 8192) == b3.blake3(d).digest(length=8192)


def test_hash_tag_key_pins(oracle):
    """hashtag.rs:188-198."""
    g = oracle.HashTag.for_profile("hashline-zk-mr1/private-block-rung-g-t24-dev/1")
    assert g.transcript.hex() == "51b7d0b0171d54b5bb45fd42c3f9369cad87894b625e0569b89fac0036d20dbe"
    assert g.column.hex() == "2295498fd6fd5e41320da717e9da89462e5c90a5b3b2d72ac496bcc157c2cd2c"
    assert g.leaf.hex() == "fe211417895c73c4a70430cb9bfb7081289ec7532f2716d2a86f609b0de54032"
    assert g.node.hex() == "8c4d2cfe7b8528d350f20dece1250c8d81596eb25d26bffda1247238f0f71fcc"
    m = oracle.HashTag.for_profile("hashline-zk-mr1/private-block-m125/1")
    assert m.transcript.hex() == "125f9b4d44ac3c46712a35419cdeda6c1428db443ccaf58da67f35b15b37291c"
    assert m.column.hex() == "d5fc391cc58eed85631b4c3dabc7d377477eb1a0a725aeccaec0f4d10061b135"
    assert m.leaf.hex() == "1dc6f7146ad501ede6d90b3071da2f3251d38137303ffcc0a6a48b7f89effe83"
    assert m.node.hex() == "798eb64ff187f6f3e8e889ac4c4742607ac71a71fa09e2944a0ecc5e8a42026b"


# --------------------------------------------------------------------------- L5: transcript
def test_l5_transcript_replay(oracle, l5):
    t, n = None, 0
    for r in l5:
        k = r[0]
        if k == "TR":
            t = oracle.Transcript(unhex(r[2])) if r[1] == "new" else oracle.Transcript(unhex(r[2]), bytes.fromhex(r[3]))
            continue
        if k == "TS":
            assert t.state.hex() == r[1]
        elif k == "TA":
            t.absorb(unhex(r[1]), data_spec(r[2]))
            assert t.state.hex() == r[3], r[:3]
        elif k == "TU":
            t.absorb_u64(unhex(r[1]), int(r[2]))
            assert t.state.hex() == r[3]
        elif k == "TF":
            t.absorb_fp(unhex(r[1]), fpv(r[2]))
            assert t.state.hex() == r[3]
        elif k == "TF2":
            v = gen_fp2(int(r[2][5:])) if r[2].startswith("fgen:") else fp2v(r[2][2:])
            t.absorb_fp2(unhex(r[1]), v)
            assert t.state.hex() == r[3], r[:3]
        elif k == "TCF":
            assert t.challenge_fp() == int(r[1]) and t.state.hex() == r[2]
        elif k == "TCF2":
            assert t.challenge_fp2() == (int(r[1]), int(r[2])) and t.state.hex() == r[3]
        elif k == "TCV":
            v = t.challenge_fp2_vec(int(r[1]))
            assert (v == fp2v(r[2])).all() and t.state.hex() == r[3]
        elif k == "TCI":
            idx = t.challenge_indices(int(r[1]), int(r[2]))
            assert (idx == fpv(r[3])).all() and t.state.hex() == r[4]
        else:
            continue
        n += 1
    assert n > 220


# --------------------------------------------------------------------------- L5: Merkle
def test_l5_merkle_records(oracle, l5):
    tags, n = {}, 0
    for r in l5:
        if r[0] == "MTAG":
            tags[r[1]] = [None if x == "-" else bytes.fromhex(x) for x in r[2:6]]
    assert tags["legacy"] == [None] * 4
    for name, prof in (("rungg", "hashline-zk-mr1/private-block-rung-g-t24-dev/1"), ("m125", "hashline-zk-mr1/private-block-m125/1")):
        t = oracle.HashTag.for_profile(prof)
        assert tags[name] == [t.transcript, t.column, t.leaf, t.node]
    for r in l5:
        if r[0] == "MB":
            nl = int(r[2])
            leaves = np.frombuffer(b"".join(oracle.blake3(i.to_bytes(8, "little")) for i in range(nl)), dtype=np.uint8).reshape(nl, 32)
            levels = oracle.merkle_build(leaves, tags[r[1]][3])
            assert bytes(levels[-1]).hex() == r[3]
            n += 1
        elif r[0] == "MP":
            path = [bytes.fromhex(x) for x in r[5].split(",")] if r[5] != "-" else []
            ok = oracle.merkle_verify_path(bytes.fromhex(r[2]), int(r[3]), bytes.fromhex(r[4]), path, tags[r[1]][3])
            assert int(ok) == int(r[6])
            n += 1
        elif r[0] == "MLEAF":
            a, b = np.frombuffer(bytes.fromhex(r[2]), np.uint8).reshape(1, 32), np.frombuffer(bytes.fromhex(r[3]), np.uint8).reshape(1, 32)
            assert bytes(oracle.salt_leaves(a, b, tags[r[1]][2])[0]).hex() == r[4]
            n += 1
        elif r[0] == "MNODE":
            assert oracle.blake3(bytes.fromhex(r[2]) + bytes.fromhex(r[3]), tags[r[1]][3]).hex() == r[4]
            n += 1
        elif r[0] == "MCOL":
            col = fpv(r[2])
            assert bytes(oracle.hash_columns(col, col.size, 1, tags[r[1]][1])[0]).hex() == r[3]
            n += 1
    assert n == 27 + 528 + 3 + 3 + 12


# --------------------------------------------------------------------------- L5: whole seeded tagged openings
def test_l5_whole_pcs_openings(oracle, l5):
    """lean_l5_export.rs:342-427: commit_zk_owned_with_tag + open_zk from ZkRng::new(seed, ..)."""
    o = oracle
    cases = {"rungg": ("hashline-zk-mr1/private-block-rung-g-t24-dev/1", 4, 4, 12, 31), "m125": ("hashline-zk-mr1/private-block-m125/1", 5, 2, 20, 32),
             "legacy": (None, 4, 4, 12, 33)}
    it = iter(l5)
    done = 0
    for r in it:
        if r[0] != "PCS":
            continue
        name = r[1]
        profile, log_cols, inv_rate, q, seed = cases[name]
        tag = o.HashTag.for_profile(profile) if profile else o.HashTag.legacy()
        p = o.PcsParams(log_cols, inv_rate, q)
        n, nn, rows = p.cols, p.enc_cols, 3
        rng = o.ZkRng(seed, b"lean-l5 pcs corpus")
        d = np.array([o.fp_from_i64(((i * 37) % 256) - 128) for i in range(rows * n)], dtype=np.uint64)
        for rr in (1, 2):
            for j in range(n):
                d[rr * n + j] = rng.fp()
        cmz = o.commit_zk(p, d, log_cols + 4, q, rng, tag)
        cmz.mask_rows, cmz.prox_mask_row = [1], 2
        assert cmz.root.hex() == r[3], name
        assert (int(r[4]), int(r[5]), int(r[6])) == (rows, nn, q)
        pt = np.array([[3000 + i * 7 + 3, 3 + i * 11 + 5] for i in range(log_cols)], dtype=np.uint64)
        e = (99991, 7)
        vp, vr = o.eval_mle_base(d[0:n], pt), o.eval_mle_base(d[n:2 * n], pt)
        one_e = o.fp2_sub((1, 0), e)
        claims = [o.ZClaim([o.ZPart(0, log_cols, one_e, pt), o.ZPart(n, log_cols, e, pt)], o.fp2_add(o.fp2_mul(one_e, vp), o.fp2_mul(e, vr)))]
        tr = o.Transcript(unhex(r[2]), tag.transcript)
        tr.absorb(b"root", cmz.root)
        op = o.open_zk(cmz, claims, tr)
        ng = int(r[7])
        assert op.group_vecs.shape[0] == ng == 1
        for g in range(ng):
            rec = next(it)
            assert rec[0] == "PCSG" and (op.group_vecs[g] == fp2v(rec[1])).all()
        rec = next(it)
        assert rec[0] == "PCSP" and (op.prox_vec == fp2v(rec[1])).all()
        for (j, col, salt, path) in op.columns:
            rec = next(it)
            assert rec[0] == "PCSC" and int(rec[1]) == j
            assert (col == fpv(rec[2])).all() and salt.hex() == rec[3]
            assert [x.hex() for x in path] == rec[4].split(",")
        rec = next(it)
        assert rec[0] == "PCSEND" and tr.state.hex() == rec[1]
        done += 1
    assert done == 3


# --------------------------------------------------------------------------- L5: the verifier on the recorded openings
def test_l5_verifier_accepts_the_recorded_openings_and_ends_in_the_recorded_state(oracle, l5):
    """lean_l5_export.rs:383-386: `verify_zk_tagged` accepts what `open_zk` wrote and leaves the transcript where the prover's is."""
    import l5_util
    for case in l5_util.pcs_cases(oracle, l5):
        tr = l5_util.start_transcript(oracle, case)
        err = oracle.verify_zk(case["params"], case["q"], case["root"], case["rows"], case["claims"], case["opening"], tr, case["tag"], case["max_log"])
        assert err is None, (case["name"], err)
        assert tr.state == case["end_state"]


def test_l5_verifier_refuses_tampered_openings_with_the_reference_messages(oracle, l5):
    """pcs.rs:1258-1335: each refusal in the order the reference makes them (lean_l5_export.rs:419-423 tampers a salt)."""
    import copy
    import l5_util
    o = oracle
    case = l5_util.pcs_cases(o, l5)[0]
    depth = (case["params"].enc_cols).bit_length() - 1

    def run(op):
        return o.verify_zk(case["params"], case["q"], case["root"], case["rows"], case["claims"], op, l5_util.start_transcript(o, case), case["tag"], case["max_log"])

    def tampered(f):
        op = copy.deepcopy(case["opening"])
        op.columns = [list(c) for c in op.columns]
        f(op)
        op.columns = [tuple(c) for c in op.columns]
        return op

    j0, j1 = case["opening"].columns[0][0], case["opening"].columns[1][0]

    def salt(op):
        b = bytearray(op.columns[0][2]); b[0] ^= 1; op.columns[0][2] = bytes(b)
    assert run(tampered(salt)) == f"pcs zk: Merkle path for column {j0} fails"

    def short_path(op):
        op.columns[2][3] = op.columns[2][3][:-1]
    assert run(tampered(short_path)) == f"pcs zk: opened column 2 carries a Merkle path of {depth - 1} entries; this commitment's tree is {depth} deep"

    def vec(op):
        op.group_vecs[0][0][0] = (int(op.group_vecs[0][0][0]) + 1) % P
    assert run(tampered(vec)) == "pcs zk: group 0: <v, c> != combined claim"

    def pad(op):  # a pad entry is outside <v, c>: the transcript moves, so the sampled columns no longer match
        op.prox_vec[-1][1] = (int(op.prox_vec[-1][1]) + 1) % P
    assert run(tampered(pad)).startswith("pcs zk: column index ")

    def col(op):  # the second column disagrees, the first column's failure would come first
        op.columns[1][1] = op.columns[1][1].copy(); op.columns[1][1][0] = (int(op.columns[1][1][0]) + 1) % P
    assert run(tampered(col)) == f"pcs zk: Merkle path for column {j1} fails"

    def drop(op):
        op.columns = op.columns[:-1]
    assert run(tampered(drop)) == "pcs zk: wrong number of columns"


def test_l5_single_column_verdicts(oracle, l5):
    """lean_l5_export.rs:399-417: 84 columns, honest and tampered, with the crate's verdict (path length and column length first)."""
    import l5_util
    o = oracle
    tags = {"rungg": o.HashTag.for_profile(l5_util.CASES["rungg"][0]), "m125": o.HashTag.for_profile(l5_util.CASES["m125"][0]), "legacy": o.HashTag.legacy()}
    seen = [0, 0]
    for name, depth, rows, root, j, col, salt, path, want in l5_util.column_records(l5):
        ok = len(path) == depth and col.size == rows
        if ok:
            none = np.zeros((0, rows, 2), dtype=np.uint64)
            ok = o.check_columns_host([col], [j], [salt], [path], root, tags[name], none, []) == [0]
        assert int(ok) == want
        seen[want] += 1
    assert seen == [72, 12]


# --------------------------------------------------------------------------- encode conformance vectors
def splitmix_fp(seed, n):
    out, s = [], seed
    for _ in range(n):
        s = (s + 0x9E3779B97F4A7C15) & M64
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        out.append((z ^ (z >> 31)) % P)
    return np.array(out, dtype=np.uint64)


def vector_inputs(v):
    """encode_conformance_tests.rs:49-84."""
    n, q, kind = int(v["n"]), int(v["q_pad"]), v["name"].split("-", 1)[1]
    msg, pad = np.zeros(n, dtype=np.uint64), np.zeros(q, dtype=np.uint64)
    if kind == "zero_msg_seeded_pad":
        pad = splitmix_fp(int(v["pad_seed"]), q)
    elif kind == "delta0":
        msg[0] = 1
    elif kind == "delta_last":
        msg[n - 1] = 1
    elif kind == "seeded":
        msg, pad = splitmix_fp(int(v["msg_seed"]), n), splitmix_fp(int(v["pad_seed"]), q)
    return msg, pad


def test_encode_conformance_vectors(oracle, golden_dir):
    g = json.load(open(os.path.join(golden_dir, "encode_vectors.json")))
    assert len(g["vectors"]) == 35
    for v in g["vectors"]:
        msg, pad = vector_inputs(v)
        assert hashlib.sha256(msg.tobytes()).hexdigest() == v["msg_sha256"]
        assert hashlib.sha256(pad.tobytes()).hexdigest() == v["pad_sha256"]
        nn = int(v["nn"])
        pows = oracle.coset_powers(7, nn)
        for max_log in {nn.bit_length() - 1, 18}:
            row = oracle.encode_row_zk(msg, pad, pows, max_log)
            assert hashlib.sha256(row.tobytes()).hexdigest() == v["encoded_sha256"], (v["name"], max_log)
        assert [int(x) for x in row[:8]] == v["encoded_first8"] and [int(x) for x in row[-8:]] == v["encoded_last8"]
        for k, want in v["encoded_probes"].items():
            assert int(row[int(k)]) == want
        if v["name"] in g["full_rows"]:
            assert [int(x) for x in row] == g["full_rows"][v["name"]]
    bad = {c["sha256"] for e in g["negative_controls"] for c in e["controls"]}
    good = {v["encoded_sha256"] for v in g["vectors"]}
    assert len(bad) == 15 and not (bad & good)


# --------------------------------------------------------------------------- L6: mle / cfs
def test_l6_mle_and_cfs_records(oracle, l6):
    o, n, mask = oracle, 0, None
    zr = o.ZkRng(61, b"lean-l6 cfs corpus")
    for r in l6:
        k = r[0]
        if k == "IE":
            assert o.interpolate_eval(fp2v(r[1]), f2(r[2])) == f2(r[3])
        elif k == "EQT":
            pt = fp2v(r[1])
            assert (o.eq_table(pt) == fp2v(r[2])).all() and (o.eq_table_msb(pt) == fp2v(r[3])).all()
        elif k == "EQP":
            pt, s = fp2v(r[1]), fp2v(r[2])
            acc = (1, 0)  # mle.rs:62-72
            for a, b in zip(pt, s):
                a, b = tuple(map(int, a)), tuple(map(int, b))
                t = o.fp2_add(o.fp2_mul(a, b), o.fp2_mul(o.fp2_sub((1, 0), a), o.fp2_sub((1, 0), b)))
                acc = o.fp2_mul(acc, t)
            assert acc == f2(r[3])
        elif k == "MLX":
            assert o.eval_mle_ext(fp2v(r[1]), fp2v(r[2])) == f2(r[3])
        elif k == "MLB":
            assert o.eval_mle_base(fpv(r[1]), fp2v(r[2])) == f2(r[3])
        elif k == "CFSM":
            nv, d = int(r[1]), int(r[2])
            mask = (zr.fp2_vec(nv * d + 2), nv, d)  # CfsMask::random draws from the same stream in order
            assert (mask[0] == fp2v(r[3])).all()
            assert o.cfs_total(*mask) == f2(r[4])
            rho = None
        elif k == "CFSV":
            rho = fp2v(r[1])
            assert o.cfs_eval(mask[0], mask[1], mask[2], rho) == f2(r[2])
        elif k == "CFSR":
            j = int(r[1])
            assert (o.cfs_round(mask[0], mask[1], mask[2], j, fp2v(r[2])) == fp2v(r[3])).all()
        elif k == "MT":
            fin, ext, rho_k = f2(r[1]), f2(r[2]), f2(r[3])
            assert o.fp2_add(fin, o.fp2_mul(rho_k, o.fp2_sub(ext, fin))) == f2(r[4])
        elif k == "EXR":
            poly = {"prod": o.POLY_PROD, "zc": o.POLY_ZC}[r[1]]
            assert (o.extension_round(poly, fp2v(r[3]), fp2v(r[4]), int(r[2])) == fp2v(r[5])).all()
        else:
            continue
        n += 1
    assert n > 300


# --------------------------------------------------------------------------- L6: whole sumchecks
def _blocks(l6):
    cur = None
    for r in l6:
        if r[0] == "SCNEW":
            if cur:
                yield cur
            cur = []
        elif cur is not None and r[0].startswith("SC"):
            cur.append(r)
    if cur:
        yield cur


def test_l6_whole_sumchecks_prover_and_verifier(oracle, l6):
    o = oracle
    honest = verdicts = 0
    for blk in _blocks(l6):
        tables = np.stack([fp2v(r[1]) for r in blk if r[0] == "SCTAB"])
        mask = next((r for r in blk if r[0] == "SCMASK"), None)
        polyname = next(r[1] for r in blk if r[0] in ("SCFIN", "SCMFIN", "SCEXT", "SCXTERM"))
        poly = {"prod": o.POLY_PROD, "zc": o.POLY_ZC}[polyname]
        # every SC ... SCEND run in the block: the verifier's verdict and transcript state
        runs, cur = [], None
        for r in blk:
            if r[0] == "SC":
                cur = {"hdr": r, "pre": None, "rounds": []}
            elif r[0] == "SCPRE":
                cur["pre"] = f2(r[1])
            elif r[0] == "SCR":
                cur["rounds"].append(fp2v(r[1]))
            elif r[0] == "SCEND":
                cur["end"] = r
                runs.append(cur)
        for run in runs:
            h = run["hdr"]
            domain, key, deg, nr, claimed = unhex(h[2]), (None if h[3] == "-" else bytes.fromhex(h[3])), int(h[4]), int(h[5]), f2(h[6])
            tv = o.Transcript(domain, key)
            if run["pre"] is not None:
                assert tv.challenge_fp2() == run["pre"]
            res, err = o.sc_verify(claimed, deg, nr, run["rounds"], tv)
            e = run["end"]
            if e[1] == "ok":
                assert res is not None and res[0] == f2(e[2])
                assert (np.array(res[1], dtype=np.uint64).reshape(-1, 2) == fp2v(e[3])).all() and tv.state.hex() == e[4]
            else:
                assert res is None and err.encode().hex() == e[2] and tv.state.hex() == e[3]
            verdicts += 1
        # the honest run, re-PROVED by the oracle from the tables (the corpus's second copy of an
        # extended run only replays the verifier on a tampered terminal: nothing to re-prove there)
        if mask is not None and not any(r[0] == "SCUNM" for r in blk):
            continue
        run = runs[0]
        h = run["hdr"]
        domain, key, deg, nr = unhex(h[2]), (None if h[3] == "-" else bytes.fromhex(h[3])), int(h[4]), int(h[5])
        n = tables.shape[1].bit_length() - 1
        tp = o.Transcript(domain, key)
        if mask is None:
            out = o.sc_prove(poly, tables, deg, tp)
            assert nr == n
        else:
            cc = tp.challenge_fp2()
            assert cc == run["pre"]
            mv, md, mco = int(mask[1]), int(mask[2]), fp2v(mask[3])
            assert md == deg
            out = o.sc_prove(poly, tables, deg, tp, mask=mco, mask_c=cc, mask_vars=mv)
            unm = [fp2v(r[2]) for r in blk if r[0] == "SCUNM"]
            assert len(unm) == n and all((out.rounds[j] == unm[j]).all() for j in range(n))
        for j in range(n):
            assert (out.masked[j] == run["rounds"][j]).all(), (h[1], j)
        fin = next(r for r in blk if r[0] in ("SCFIN", "SCMFIN", "SCEXT"))
        assert (out.finals == fp2v(fin[2])).all()
        if fin[0] == "SCEXT":  # masked + one extension round (argument.rs private slot form)
            exts = fp2v(fin[3])
            sk = o.extension_round(poly, out.finals, exts, deg)
            gk = o.cfs_round(mco, mv, md, n, out.challenges)
            sk = np.array([o.fp2_add(tuple(map(int, s)), o.fp2_mul(cc, tuple(map(int, g)))) for s, g in zip(sk, gk)], dtype=np.uint64)
            assert nr == n + 1 and (sk == run["rounds"][n]).all()
            tp.absorb_fp2(b"sc-round", sk)
            tp.challenge_fp2()
        assert tp.state.hex() == run["end"][-1], h[1]
        # s(1) recovery gives the same messages (sumcheck/rounds.rs:94-147)
        if mask is None and n >= 1 and deg >= 1:
            t2 = o.Transcript(domain, key)
            out2 = o.sc_prove(poly, tables, deg, t2, recover_one=True)
            assert (out2.rounds == out.rounds).all() and t2.state == tp.state
        honest += 1
    assert honest == 15 and verdicts >= 171


# ----------------------------------------------------------------------------- L11: the slots of a real W16R2 block core
@pytest.fixture(scope="module")
def l11(golden_dir):
    import l11_util

    return l11_util.load(golden_dir)


def _eq_point(o, point, s):
    """mle.rs:62-71"""
    acc = (1, 0)
    for a, b in zip(point, s):
        t = o.fp2_add(o.fp2_mul(a, b), o.fp2_mul(o.fp2_sub((1, 0), a), o.fp2_sub((1, 0), b)))
        acc = o.fp2_mul(acc, t)
    return acc


def test_l11_head_replays_to_the_logup_challenges(oracle, l11):
    """`verify_core`'s head (protocol.rs:2827-2837) from the recorded header state: absorb the `A` root, `M`, draw beta,
    gamma, alpha, absorb the `H` root; the tag constants are gamma times the table tags."""
    o, h = oracle, l11["head"]
    r = h["roots"]
    tr = o.Transcript.from_state(*h["head"], key=h["key"])
    for label, root, rows in ((b"A", r["a_root"], r["a_rows"]),):
        tr.absorb(label, root)
        tr.absorb_u64(b"rows", rows)
        tr.absorb_u64(b"log-cols", r["log_cols"])
    tr.absorb(b"M", r["mask_root"])
    assert tr.challenge_fp2() == h["beta"]
    gamma = tr.challenge_fp2()
    assert gamma == h["gamma"]
    assert tr.challenge_fp2() == h["alpha"]
    tr.absorb(b"H", r["h_root"])
    tr.absorb_u64(b"rows", r["h_rows"])
    tr.absorb_u64(b"log-cols", r["log_cols"])
    assert (tr.state, tr.counter) == h["headend"]
    # the three tags are gamma times the table tags (tables_attn.rs:49,70,77: TAG_EXP 129, TAG_U8 133, TAG_ACT 134)
    for name, tag in (("g_u8", 133), ("g_exp", 129), ("g_act", 134)):
        assert o.fp2_mul_base(gamma, tag) == h[name]


def test_l11_slot_graphs_evaluate_to_the_reference_value(oracle, l11):
    """Every slot's expression graph, WITH the recorded coefficient values, evaluated at the recorded terminal values by
    the oracle's interpreter and by the independent Python walk: the reference's own `poly(vals)` (slot_ir.rs:352-377,
    the `ir.eval(&vals) == (def.poly)(&vals)` assertion of lean_l11_export_tests.rs:243)."""
    from intelligenceregulation_b200 import backend
    import ir_util
    import l11_util

    o = oracle
    for s in l11["slots"]:
        assert len(s["vals"]) == s["n_tabs"] == s["ir_counts"][0] == len(s["tabs"])
        prog, desc = l11_util.build_program(backend, s)
        assert ir_util.py_eval(desc, s["vals"]) == s["pv"], s["slot"]
        cf = prog.coef_array()
        o.ir_set(prog.words(), prog.n_nodes, prog.n_terms)
        assert o.poly_eval(o.POLY_IR, np.array(s["vals"], dtype=np.uint64), cf if cf.size else None) == s["pv"], s["slot"]


def test_l11_verify_arm_of_every_slot(oracle, l11):
    """`run_slot`'s VERIFY arm (argument.rs:1434-1468) recomputed from the recorded proof: the slot challenge `c`, the claimed
    sum with its hosted terms, the sumcheck verifier through every recorded round to `fin` and `rho`, the terminal values of
    eq tables (`sel * eq_point`) and public tables (`sel * mle(pub)(rho)`), the mask value `g = (fin - poly(vals)) / c`, the
    transcript state after `pb-term`; and the chain between slots (a definition only squeezes)."""
    o, key = oracle, l11["head"]["key"]
    scalars = []
    prev = l11["head"]["headend"]
    for s in l11["slots"]:
        # the definition's draws: squeezes only, from where the previous slot (or the head) ended
        tr = o.Transcript.from_state(*prev, key=key)
        assert [tr.challenge_fp2() for _ in s["draws"]] == s["draws"]
        assert (tr.state, tr.counter) == s["trb"]
        n, ext, deg = s["n"], s["ext"], s["degree"]
        tr.absorb_u64(b"pb-slot", s["slot"])
        c = tr.challenge_fp2()
        assert c == s["c"]
        tr.absorb_fp2(b"pb-scalar", np.array([s["scalar"]], dtype=np.uint64))
        claimed = s["scalar"]
        for hs, coef in s["hosted"]:
            claimed = o.fp2_add(claimed, o.fp2_mul(coef, scalars[hs]))
        assert claimed == s["claimed"]
        rounds = [np.array(r, dtype=np.uint64) for r in s["rounds"]]
        got, err = o.sc_verify(claimed, deg, n + ext, rounds, tr)
        assert err is None, (s["slot"], err)
        fin, rho_full = got
        assert fin == s["fin"] and [tuple(map(int, r)) for r in rho_full] == s["rho_full"]
        rho, es = s["rho_full"][:n], s["rho_full"][n:]
        sel = (1, 0)
        for e in es:
            sel = o.fp2_mul(sel, o.fp2_sub((1, 0), e))
        k = 0
        for i, t in enumerate(s["tabs"]):
            if t[0] == "eq":
                want = o.fp2_mul(sel, _eq_point(o, t[2], rho[t[1]:t[1] + len(t[2])]))
            elif t[0] == "pub":
                assert len(t[2]) == t[1] == 1 << n
                want = o.fp2_mul(sel, o.eval_mle_ext(np.array(t[2], dtype=np.uint64), np.array(rho, dtype=np.uint64)))
            elif t[0] == "pubv":
                want = o.fp2_mul(sel, t[2])
            else:
                assert t[1] == k
                want = s["terms_vals"][k]
                k += 1
            assert want == s["vals"][i], (s["slot"], i, t[0])
        assert k == s["n_priv"] == len(s["terms_vals"])
        assert o.fp2_mul(o.fp2_sub(fin, s["pv"]), o.fp2_inv(c)) == s["g"]
        tr.absorb_fp2(b"pb-term", np.array(s["terms_vals"], dtype=np.uint64).reshape(-1, 2))
        assert (tr.state, tr.counter) == s["tra"], s["slot"]
        scalars.append(s["scalar"])
        prev = s["tra"]


def test_l11_lookup_denominator_rule(oracle, l11):
    """The table-indexed helper rule of protocol.rs:1125-1230 as the slot graphs record it with real values: a helper
    constraint's affine node is `alpha - (word + cst + g_tag)` (konst `alpha - (cst + g_tag)`, coefficient -1 on the looked
    word, `cst` a small integer offset), and the oracle's inverse table holds `1 / (alpha - (v + g_tag))` at `v = word + cst`.
    For every such node of the corpus, inverting the node's value at a word reproduces the oracle's table entry."""
    o, h = oracle, l11["head"]
    seen = {}
    for s in l11["slots"]:
        for n in s["nodes"]:
            if n[0] != "affine" or len(n[2]) != 1 or n[2][0][0][0] != (P - 1, 0):
                continue
            konst = n[1][0]
            for tag in ("g_u8", "g_exp", "g_act"):
                cst = o.fp2_sub(o.fp2_sub(h["alpha"], h[tag]), konst)
                if cst[1] != 0 or not (cst[0] < 4096 or P - cst[0] < 4096):
                    continue
                off = cst[0] if cst[0] < 4096 else cst[0] - P
                tab, absent = o.lookup_inverse_table(h["alpha"], h[tag], 8192)
                for word in (0, 1, 77, 255, 4000):
                    if not 0 <= word + off < 8192:
                        continue
                    den = o.fp2_sub(konst, (word, 0))
                    assert not absent[word + off] and tuple(map(int, tab[word + off])) == o.fp2_inv(den)
                seen[tag] = seen.get(tag, 0) + 1
    assert seen.get("g_u8", 0) > 0, seen
