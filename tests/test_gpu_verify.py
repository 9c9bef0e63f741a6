"""The verifier's per-column checks on the device (`hl_b200_verify_columns`, pcs.rs:1303-1331) against the reference's own verdicts:
the 84 single columns of the L5 corpus, honest and tampered; the three whole recorded openings through the restated verifier with
the device as its column checker (both ways of giving the expected values); a block-sized opening (2^16 columns at rate 1/2,
2,500 rows, 280 opened columns) with tampered columns of every kind, verdict by verdict against the host body.  Byte and integer
work: exact."""
import copy
import os

import numpy as np
import pytest

import l5_util

pytestmark = pytest.mark.gpu
P = 0xFFFFFFFF00000001


@pytest.fixture(scope="module")
def dev():
    from intelligenceregulation_b200 import backend

    d = backend.B200Backend(device=0)
    yield d
    d.ctx.close()


@pytest.fixture(scope="module")
def l5(golden_dir):
    return [l.rstrip("\n").split(" ") for l in open(os.path.join(golden_dir, "l5_corpus.txt")) if l.strip() and not l.startswith("#")]


def device_checker(dev, case_params, max_log, o, form):
    """the `check_columns` hook of the restated verifier, on the device"""
    def check(cols, idx, salts, paths, root, tag, rhos, vecs, encoded_vecs):
        cols = np.stack([np.asarray(c, dtype=np.uint64) for c in cols])
        salts = np.frombuffer(b"".join(salts), dtype=np.uint8).reshape(len(idx), 32)
        paths = np.frombuffer(b"".join(b"".join(p) for p in paths), dtype=np.uint8).reshape(len(idx), -1, 32)
        if form in ("store", "one_call"):
            v = dev.check_opening_columns(case_params.log_cols, case_params.inv_rate, o.coset_powers(7, case_params.enc_cols), max_log, cols, idx, salts, paths,
                                          root, tag.column, tag.leaf, tag.node, rhos, vecs, one_call=form == "one_call")
            assert v is not None, dev.ctx.declines
            return [int(x) for x in v]
        wants = np.array([[[int(e[0][int(j)]), int(e[1][int(j)])] for j in idx] for e in encoded_vecs], dtype=np.uint64)
        return [int(x) for x in dev.ctx.verify_columns(cols, idx, salts, paths, root, tag.column, tag.leaf, tag.node, rhos=rhos, wants=wants)]
    return check


def test_l5_single_column_verdicts_on_the_device(dev, oracle, l5):
    o = oracle
    tags = {"rungg": o.HashTag.for_profile(l5_util.CASES["rungg"][0]), "m125": o.HashTag.for_profile(l5_util.CASES["m125"][0]), "legacy": o.HashTag.legacy()}
    seen = [0, 0]
    # records of one (profile, shape) go to the device together; the two length refusals are the caller's (pcs.rs:1258-1263, 1310-1312)
    batches = {}
    for rec in l5_util.column_records(l5):
        name, depth, rows, root, j, col, salt, path, want = rec
        if len(path) != depth or col.size != rows:
            assert want == 0
            seen[0] += 1
            continue
        batches.setdefault((name, depth, rows, root), []).append(rec)
    for (name, depth, rows, root), recs in batches.items():
        cols = np.stack([r[5] for r in recs])
        idx = np.array([r[4] for r in recs], dtype=np.uint64)
        salts = np.frombuffer(b"".join(r[6] for r in recs), dtype=np.uint8).reshape(len(recs), 32)
        paths = np.frombuffer(b"".join(b"".join(r[7]) for r in recs), dtype=np.uint8).reshape(len(recs), depth, 32)
        t = tags[name]
        v = dev.ctx.verify_columns(cols, idx, salts, paths, root, t.column, t.leaf, t.node)
        for r, got in zip(recs, v):
            assert int(got == 0) == r[8]
            seen[r[8]] += 1
    assert seen == [72, 12]


@pytest.mark.parametrize("form", ["wants", "store", "one_call"])
def test_l5_recorded_openings_verify_with_the_device_as_column_checker(dev, oracle, l5, form):
    o = oracle
    for case in l5_util.pcs_cases(o, l5):
        chk = device_checker(dev, case["params"], case["max_log"], o, form)
        tr = l5_util.start_transcript(o, case)
        err = o.verify_zk(case["params"], case["q"], case["root"], case["rows"], case["claims"], case["opening"], tr, case["tag"], case["max_log"], check_columns=chk)
        assert err is None, (case["name"], err)
        assert tr.state == case["end_state"]
        # lean_l5_export.rs:419-423: a flipped salt bit is refused, with the host body's message
        for at, what in ((0, "salt"), (3, "col"), (5, "path")):
            bad = copy.deepcopy(case["opening"])
            j, col, salt, path = bad.columns[at]
            if what == "salt":
                salt = bytes([salt[0] ^ 1]) + salt[1:]
            elif what == "col":
                col = col.copy()
                col[1] = (int(col[1]) + 1) % P
            else:
                path = [path[0], bytes([path[1][0] ^ 1]) + path[1][1:]] + path[2:]
            bad.columns[at] = (j, col, salt, path)
            args = (case["params"], case["q"], case["root"], case["rows"], case["claims"], bad)
            host = o.verify_zk(*args, l5_util.start_transcript(o, case), case["tag"], case["max_log"])
            got = o.verify_zk(*args, l5_util.start_transcript(o, case), case["tag"], case["max_log"], check_columns=chk)
            assert host is not None and got == host


def test_block_sized_opening_with_every_kind_of_tampered_column(dev, oracle):
    """2^16 columns at rate 1/2, 2,500 rows, 280 opened columns (the 8B block commitment's shape): the device's verdicts equal the host
    body's on an honest opening and on one whose columns are damaged in a word, the salt, the path, the position, or only in what a
    combination must equal."""
    o = oracle
    log_cols, ir, rows, q, checks = 16, 2, 2500, 280, 280
    n, nn = 1 << log_cols, (1 << log_cols) * ir
    depth = log_cols + 1
    tag = o.HashTag.for_profile("hashline-zk-mr1/private-block-m125/1")
    rs = np.random.default_rng(5)
    data = rs.integers(0, P, rows * n, dtype=np.uint64)
    rng = o.ZkRng(9, b"verify-block")
    pads, salts = rng.fp_vec(rows * q), rng.salts(nn)
    pows = o.coset_powers(7, nn)
    store, _, levels = dev.try_commit_zk_tree(log_cols, ir, data, pads, pows, 18, tag.column, salts, tag.leaf, tag.node, want_leaves=False)
    root = bytes(levels[-1])
    # three combined row weights: one living on a few rows, two dense
    rhos = np.zeros((3, rows, 2), dtype=np.uint64)
    rhos[0, 7:19] = rs.integers(0, P, (12, 2), dtype=np.uint64)
    rhos[1:] = rs.integers(0, P, (2, rows, 2), dtype=np.uint64)
    vecs = store.fold_rows_with_pads(rhos)
    idx = rs.integers(0, nn, checks, dtype=np.uint64)
    idx[1] = idx[0]  # a position sampled twice
    cols = store.columns(idx)
    store.free()
    paths = np.stack([np.stack([np.frombuffer(x, dtype=np.uint8) for x in o.merkle_path(levels, nn, int(j))]) for j in idx])
    sl = np.stack([salts[int(j)] for j in idx])
    v = dev.check_opening_columns(log_cols, ir, pows, 18, cols, idx, sl, paths, root, tag.column, tag.leaf, tag.node, rhos, vecs)
    assert v is not None and (v == 0).all()
    v = dev.check_opening_columns(log_cols, ir, pows, 18, cols, idx, sl, paths, root, tag.column, tag.leaf, tag.node, rhos, vecs, one_call=False)
    assert v is not None and (v == 0).all()
    # the host body on a sample of the honest columns (the whole of it takes a pure-Python minute)
    enc_vecs = [(o.encode_row_zk(x[:n, 0], x[n:, 0], pows, 18), o.encode_row_zk(x[:n, 1], x[n:, 1], pows, 18)) for x in vecs]
    pl = [[bytes(p) for p in paths[c]] for c in range(checks)]
    assert o.check_columns_host([cols[c] for c in (0, 1, 279)], idx[[0, 1, 279]], [bytes(sl[c]) for c in (0, 1, 279)], [pl[c] for c in (0, 1, 279)], root, tag, rhos,
                                enc_vecs) == [0, 0, 0]
    # damage
    c2, s2, p2, i2 = cols.copy(), sl.copy(), paths.copy(), idx.copy()
    c2[3, rows - 1] = (int(c2[3, rows - 1]) + 1) % P      # a word of the column
    s2[10, 31] ^= 0x80                                     # the salt
    p2[20, depth - 1, 5] ^= 1                              # the sibling below the root
    p2[21, 0, 0] ^= 1                                      # the sibling next to the leaf
    i2[30] ^= 1                                            # the neighbouring position
    bad = [3, 10, 20, 21, 30]
    v = dev.check_opening_columns(log_cols, ir, pows, 18, c2, i2, s2, p2, root, tag.column, tag.leaf, tag.node, rhos, vecs)
    assert sorted(np.nonzero(v)[0].tolist()) == bad and all(v[c] == 1 for c in bad)
    host = o.check_columns_host([c2[c] for c in bad], i2[bad], [bytes(s2[c]) for c in bad], [[bytes(p) for p in p2[c]] for c in bad], root, tag, rhos, enc_vecs)
    assert host == [1] * 5
    # honest columns against a damaged clear vector: every column disagrees with that vector and only with it
    for g in range(3):
        v2 = vecs.copy()
        v2[g, 5, 1] = (int(v2[g, 5, 1]) + 1) % P
        v = dev.check_opening_columns(log_cols, ir, pows, 18, cols, idx, sl, paths, root, tag.column, tag.leaf, tag.node, rhos, v2)
        assert (v == 2 + g).all()
    e2 = [(a.copy(), b.copy()) for a, b in enc_vecs]
    e2[1][1][int(idx[0])] ^= np.uint64(1)
    assert o.check_columns_host([cols[0]], idx[:1], [bytes(sl[0])], [pl[0]], root, tag, rhos, e2) == [3]
    # the expected values handed over instead of the vectors' store: the same verdicts, and a single wrong value is found where it is
    wants = np.array([[[int(e[0][int(j)]), int(e[1][int(j)])] for j in idx] for e in enc_vecs], dtype=np.uint64)
    assert (dev.ctx.verify_columns(cols, idx, sl, paths, root, tag.column, tag.leaf, tag.node, rhos=rhos, wants=wants) == 0).all()
    wants[2, 100, 0] ^= np.uint64(1)
    v = dev.ctx.verify_columns(cols, idx, sl, paths, root, tag.column, tag.leaf, tag.node, rhos=rhos, wants=wants)
    assert v[100] == 4 and np.count_nonzero(v) == 1


def test_refusals(dev):
    """bad arguments are refused on the host: nothing is launched"""
    from intelligenceregulation_b200 import backend
    cols = np.zeros((2, 3), dtype=np.uint64)
    idx = np.zeros(2, dtype=np.uint64)
    salts = np.zeros((2, 32), dtype=np.uint8)
    paths = np.zeros((2, 4, 32), dtype=np.uint8)
    rhos = np.zeros((1, 3, 2), dtype=np.uint64)
    with pytest.raises(backend.DeviceError):
        dev.ctx.verify_columns(cols, idx, salts, paths, bytes(32), None, None, None, rhos=rhos)  # neither expected values nor a store
    with pytest.raises(backend.DeviceError):
        dev.ctx.verify_columns(cols, idx, salts, np.zeros((2, 41, 32), dtype=np.uint8), bytes(32), None, None, None)
    # no weights at all: the hash and path part alone
    v = dev.ctx.verify_columns(cols, idx, salts, paths, bytes(32), None, None, None)
    assert (v == 1).all()
    # the one-call form: a position beyond the encoding, and a pad count the encoder cannot take, are declines (None), nothing is compared
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
    import hl_oracle as o
    pows = o.coset_powers(7, 32)
    vecs = np.zeros((1, 16 + 4, 2), dtype=np.uint64)
    declines = len(dev.ctx.declines)
    far = np.array([5, 32], dtype=np.uint64)
    assert dev.check_opening_columns(4, 2, pows, 6, cols, far, salts, paths[:, :1], bytes(32), None, None, None, rhos, vecs) is None
    wide = np.zeros((1, 16 + 17, 2), dtype=np.uint64)  # n + q > nn
    assert dev.check_opening_columns(4, 2, pows, 6, cols, idx, salts, paths[:, :1], bytes(32), None, None, None, rhos, wide) is None
    assert len(dev.ctx.declines) == declines + 2
    # and the same shapes accepted: every column fails its (all-zero) path, verdict 1
    v = dev.check_opening_columns(4, 2, pows, 6, cols, idx, salts, paths[:, :1], bytes(32), None, None, None, rhos, vecs)
    assert v is not None and (v == 1).all()
