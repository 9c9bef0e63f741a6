"""The masking commitment M on the device == the CPU restatement of hashline/src/zk.rs:447-656 (mask_commit_tagged,
mask_open), word for word: coefficients, encoded rows (through the opened columns and the leaves), tree, product
polynomial, proximity combination; and the restated verifier (zk.rs:658-760) accepts the opening assembled from the
device's parts.  The restatement of this part has no reference vector to pin it (see its header); its primitives do."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from intelligenceregulation_b200 import backend

    c = backend.Context(0)
    yield c
    c.close()


def _functionals(o, mc, specs, count, seed):
    fr, fs = o.ZkRng(seed, b"mask-functionals"), []
    for i in range(count):
        terms, val = [], (0, 0)
        for row in sorted({i % len(specs), (3 * i + 1) % len(specs)}):
            w = fr.fp2_vec(specs[row][0] * specs[row][1] + 2)
            for j in range(len(w)):
                val = o.fp2_add(val, o.fp2_mul((int(w[j, 0]), int(w[j, 1])), (int(mc.masks[row][j, 0]), int(mc.masks[row][j, 1]))))
            terms.append((row, w))
        fs.append((val, terms))
    return fs


@pytest.mark.parametrize("specs,log_msg,log_dom,q", [
    ([(5, 3), (9, 2), (7, 5)], 9, 12, 256),                               # the reference's constants (zk.rs:391-393)
    ([(21, 3)] * 12 + [(19, 5)] * 8 + [(14, 2)] * 4, 9, 12, 256),         # 24 masks: a block's 52 rows
    ([(3, 2)], 8, 9, 100), ([(20, 4), (22, 7)], 10, 13, 256), ([(30, 6)] * 3, 11, 17, 512),
])
def test_commit_and_open(ctx, oracle, specs, log_msg, log_dom, q):
    from intelligenceregulation_b200 import backend

    o = oracle
    m, dom, S = 1 << log_msg, 1 << log_dom, len(specs)
    tag = o.HashTag.for_profile("hashline-zk-mr1/b200-mask/1")
    mc = o.mask_commit(specs, o.ZkRng(11 + S, b"mask"), tag, log_msg, log_dom, q)
    coef_rows = np.stack([mc.b[0], mc.b[1], mc.u[0], mc.u[1]])
    dm = backend.mask_commit(ctx, mc.msgs, coef_rows, o.coset_powers(7, dom), tag.column, log_msg, log_dom)
    assert dm is not None and (dm.rows, dm.n, dm.nn) == (2 * S + 4, 2 * m, dom)
    assert (dm.a_coefs == mc.a_coefs).all()
    assert (dm.leaves == o.hash_columns(mc.encoded, 2 * S + 4, dom, tag.column)).all()
    levels = dm.merkle(mc.salts, tag.leaf, tag.node)
    assert (levels == mc.levels).all()
    # the opening, part by part, on one transcript (zk.rs:618-656)
    fs = _functionals(o, mc, specs, 5, 3)
    tr0 = o.Transcript(b"mask-open", tag.transcript)
    want_q, want_prox, want_cols, ws, rs = o.mask_open(mc, fs, tr0.clone(), log_msg, log_dom, q)
    tr = tr0.clone()
    theta = tr.challenge_fp2()
    ws_d, _ = o.mask_combined_weights(specs, fs, theta, m)  # the functionals' weights are the caller's host logic
    qv = dm.open_q(ws_d)
    assert (qv == want_q).all()
    tr.absorb_fp2(b"mask-q", qv)
    prox = dm.prox(tr.challenge_fp2_vec(2 * S + 2))
    assert (prox == want_prox).all()
    tr.absorb_fp2(b"mask-prox", prox)
    idx = tr.challenge_indices(q, dom)
    cols = dm.columns(idx)
    assert all((cols[i] == want_cols[i][1]).all() for i in range(len(idx)))
    opening = (qv, prox, [(int(j), cols[i], bytes(mc.salts[int(j)]), o.merkle_path(levels, dom, int(j))) for i, j in enumerate(idx)])
    assert o.mask_verify(bytes(levels[-1]), specs, fs, opening, tr0.clone(), tag, log_msg, log_dom, q) is None
    dm.free()


def test_shapes_the_device_declines(ctx, oracle):
    from intelligenceregulation_b200 import backend

    z = np.zeros((2, 1 << 12), dtype=np.uint64)
    assert backend.mask_commit(ctx, z, np.zeros((4, 1 << 13), dtype=np.uint64), oracle.coset_powers(7, 1 << 14), None, 12, 14) is None
    assert ctx.declines and ctx.declines[-1][0] == "b200 mask commit"
