"""The CPU restatement of the masking commitment M (hashline/src/zk.rs:447-760): what the reference's own tests of it
assert (zk.rs tests, zk_f12_tests.rs) — an honest opening verifies; a wrong functional value, a tampered product polynomial,
proximity vector, column or path does not; the combined weights start at theta^1.  Small masks keep this in a second."""
import numpy as np


def _setup(o, specs, seed=5):
    tag = o.HashTag.for_profile("hashline-zk-mr1/mask-cpu/1")
    mc = o.mask_commit(specs, o.ZkRng(seed, b"mask"), tag)
    fr, fs = o.ZkRng(seed + 1, b"f"), []
    for i in range(3):
        row = i % len(specs)
        w = fr.fp2_vec(specs[row][0] * specs[row][1] + 2)
        val = (0, 0)
        for j in range(len(w)):
            val = o.fp2_add(val, o.fp2_mul((int(w[j, 0]), int(w[j, 1])), (int(mc.masks[row][j, 0]), int(mc.masks[row][j, 1]))))
        fs.append((val, [(row, w)]))
    return tag, mc, fs


def test_honest_opening_verifies_and_tampering_does_not(oracle):
    o = oracle
    specs = [(4, 3), (6, 2)]
    tag, mc, fs = _setup(o, specs)
    assert mc.encoded.shape == (2 * len(specs) + 4, 4096) and mc.a_coefs.shape == (4, 512)
    # b sums to zero over G_512: coefficient 0 plus coefficient 512 (zk.rs:480-481)
    assert o.fp_add(int(mc.b[0][0]), int(mc.b[0][512])) == 0 and o.fp_add(int(mc.b[1][0]), int(mc.b[1][512])) == 0
    tr = o.Transcript(b"m", tag.transcript)
    q, prox, cols, ws, rs = o.mask_open(mc, fs, tr.clone())
    assert len(cols) == o.MASK_Q and q.shape == (1024, 2) and prox.shape == (1024, 2)
    assert o.mask_verify(mc.root, specs, fs, (q, prox, cols), tr.clone(), tag) is None
    # the same opening under another profile's keys, or under no keys, fails
    assert o.mask_verify(mc.root, specs, fs, (q, prox, cols), tr.clone(), o.HashTag.for_profile("other/1")) is not None
    # a false functional
    fs_bad = [(o.fp2_add(fs[0][0], (1, 0)), fs[0][1])] + fs[1:]
    assert "sum" in o.mask_verify(mc.root, specs, fs_bad, (q, prox, cols), tr.clone(), tag)
    # a tampered proximity vector moves the column challenge; with the columns re-drawn for it, the column check refuses
    p2 = prox.copy()
    p2[700, 1] ^= 1
    assert o.mask_verify(mc.root, specs, fs, (q, p2, cols), tr.clone(), tag) is not None
    # a tampered column word: Merkle path fails
    c2 = [(j, c.copy(), s, p) for j, c, s, p in cols]
    c2[5][1][2] ^= 1
    assert "Merkle" in o.mask_verify(mc.root, specs, fs, (q, prox, c2), tr.clone(), tag)


def test_weights_start_at_theta(oracle):
    o = oracle
    specs = [(2, 2)]
    w = np.array([[1, 0]] * 6, dtype=np.uint64)
    theta = (3, 0)
    ws, v = o.mask_combined_weights(specs, [((5, 0), [(0, w)]), ((7, 0), [(0, w)])], theta, 512)
    assert tuple(int(x) for x in ws[0, 0]) == (3 + 9, 0) and v == (5 * 3 + 7 * 9, 0) and not ws[0, 6:].any()
