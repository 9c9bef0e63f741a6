"""Device == CPU oracle for the Ligero commitment and its store, through the C ABI.

Modelled on the reference's hashline/tests/zk60_metal_commit.rs (field probe :69-89, plain
commit over nine shapes :92-134, hiding + keyed commit with complete opening bytes :157-219)
and on zkp-core's encode conformance vectors.  Integer work: every comparison is bit-exact.
"""
import hashlib
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

P = 0xFFFFFFFF00000001
M64 = (1 << 64) - 1


def rnd(seed, n):
    """zk60_metal_commit.rs:44-56 (SplitMix64 words mod p)."""
    s = (seed ^ 0x9E3779B97F4A7C15) & M64
    i = np.arange(1, n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(s) + i * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z % np.uint64(P)


def rnd2(seed, n):
    return np.stack([rnd(seed, n), rnd(seed ^ 0x55, n)], axis=1)


@pytest.fixture(scope="module")
def dev():
    from intelligenceregulation_b200 import backend

    b = backend.B200Backend()
    yield b
    b.ctx.close()


def test_m0_field_ops_match_the_cpu_on_edges_and_random_values(dev, oracle):
    edges = [0, 1, 2, P - 1, P - 2, 1 << 32, (1 << 32) - 1, (1 << 32) + 1, 1 << 63, (1 << 63) + 5, 0xFFFFFFFF, P >> 1]
    a = np.array([x for x in edges for _ in edges] + list(rnd(1, 100_000)), dtype=np.uint64)
    b = np.array([y for _ in edges for y in edges] + list(rnd(2, 100_000)), dtype=np.uint64)
    got = dev.ctx.probe_field(a, b)
    ai, bi = a.astype(object), b.astype(object)
    assert (got[:, 0].astype(object) == (ai + bi) % P).all()
    assert (got[:, 1].astype(object) == (ai - bi) % P).all()
    assert (got[:, 2].astype(object) == (ai * bi) % P).all()
    for i in range(0, 200):
        assert int(got[i, 2]) == oracle.fp_mul(int(a[i]), int(b[i]))


# (log_cols, inv_rate, rows): rows * 8 bytes per column = 1 .. 17 BLAKE3 chunks (zk60_metal_commit.rs:92-93)
SHAPES = [(3, 4, 1), (4, 4, 5), (6, 4, 8), (8, 2, 127), (8, 4, 128), (8, 4, 129), (10, 4, 300), (12, 4, 1100), (6, 8, 2049)]


@pytest.mark.parametrize("fast", [True, False])
def test_m1_plain_commit_leaves_root_columns_and_folds_match_the_cpu(dev, oracle, fast):
    dev.ctx.set_encoder(fast)
    for si, (log_cols, ir, rows) in enumerate(SHAPES):
        n, nn = 1 << log_cols, (1 << log_cols) * ir
        data = rnd(10 + si, rows * n)
        enc = oracle.encode_rows_plain(data, rows, n, nn, 16)
        got = dev.try_commit(log_cols, ir, data, 16)
        assert got is not None, dev.ctx.declines
        store, leaves = got
        want_leaves = oracle.hash_columns(enc, rows, nn)
        assert (leaves == want_leaves).all(), f"shape {si}: leaves"
        levels = store.merkle(None, None, None)
        assert (levels == oracle.merkle_build(want_leaves)).all(), f"shape {si}: tree"
        idx = np.array([j % nn for j in (0, 1, nn // 2, nn - 1, 7 % nn, (nn // 3) | 1, 0)], dtype=np.uint64)
        assert (store.columns(idx) == oracle.gather_columns(enc, rows, nn, idx)).all(), f"shape {si}: columns"
        rhos = np.stack([rnd2(100 + si, rows), rnd2(200 + si, rows)])
        assert (store.fold_rows(rhos) == oracle.fold_rows(enc, rows, n, nn, ir, rhos)).all(), f"shape {si}: folds"
        store.free()
    dev.ctx.set_encoder(True)


def _claims(o, rows, log_cols, seed):
    """zk60_metal_commit.rs:138-155."""
    n = 1 << log_cols
    r = rnd2(seed, log_cols)
    e = (99991, 7)
    return [
        o.ZClaim([o.ZPart(0, log_cols, o.fp2_sub((1, 0), e), r), o.ZPart((rows - 3) * n, log_cols, e, r)], (0, 0)),
        o.ZClaim([o.ZPart((rows - 2) * n, log_cols, (1, 0), np.zeros((0, 2), dtype=np.uint64))], (0, 0)),
    ]


@pytest.mark.parametrize("keyed", [False, True])
@pytest.mark.parametrize("fast", [True, False])
def test_m1_zk_commit_and_opening_bytes_match_the_cpu(dev, oracle, keyed, fast):
    o = oracle
    dev.ctx.set_encoder(fast)
    tag = o.HashTag.for_profile("hashline-zk-mr1/metal-test/1") if keyed else o.HashTag.legacy()
    cases = 0
    for si, (log_cols, ir, rows0) in enumerate(SHAPES):
        rows = max(rows0, 4)
        n, nn = 1 << log_cols, (1 << log_cols) * ir
        q = 12 if log_cols == 3 else 8  # q > n: the interleaved pad branch (encode_buffer.rs:56-64)
        if n + q > nn:
            continue
        p = o.PcsParams(log_cols, ir, 8)
        data = rnd(500 + si, rows * n)
        cpu = o.commit_zk(p, data, 16, q, o.ZkRng(42 + si, b"metal-zk-test"), tag)
        # the device commitment: the same draws in the same order, then the backend hook (pcs.rs:782-817)
        rng = o.ZkRng(42 + si, b"metal-zk-test")
        pads, salts = rng.fp_vec(rows * q), rng.salts(nn)
        got = dev.try_commit_zk_keyed(log_cols, ir, data, pads, o.coset_powers(7, nn), 16, tag.column)
        assert got is not None, dev.ctx.declines
        store, leaves = got
        assert (leaves == cpu.leaves).all(), f"shape {si}: unsalted leaves"
        levels = store.merkle(salts, tag.leaf, tag.node)
        assert bytes(levels[-1]) == cpu.root, f"shape {si}: salted root"
        assert (levels == cpu.levels).all()
        assert (dev.ctx.merkle(leaves, salts, tag.leaf, tag.node) == cpu.levels).all()
        # the commitment and its salted tree in one call
        st2, leaves2, levels2 = dev.try_commit_zk_tree(log_cols, ir, data, pads, o.coset_powers(7, nn), 16, tag.column, salts, tag.leaf, tag.node)
        assert (leaves2 == cpu.leaves).all() and (levels2 == cpu.levels).all()
        st2.free()
        st3, none, levels3 = dev.try_commit_zk_tree(log_cols, ir, data, pads, o.coset_powers(7, nn), 16, tag.column, salts, tag.leaf, tag.node,
                                                    want_leaves=False)
        assert none is None and (levels3 == cpu.levels).all()
        st3.free()
        for c in (cpu,):
            c.mask_rows, c.prox_mask_row = [rows - 3, rows - 2], rows - 1
        cl = _claims(o, rows, log_cols, 900 + si)
        t1, t2 = o.Transcript(b"metal-open"), o.Transcript(b"metal-open")
        o1 = o.open_zk(cpu, cl, t1)
        o2 = o.open_zk(cpu, cl, t2, fold=store.fold_rows_with_pads, columns=store.columns)
        assert o1.to_bytes() == o2.to_bytes(), f"shape {si}: opening bytes"
        assert t1.challenge_fp2() == t2.challenge_fp2()
        # the split form (fold_rows in batches, pads folded apart) gives the same vectors
        rhos = np.stack([rnd2(7 + si, rows), rnd2(8 + si, rows), rnd2(9 + si, rows)])
        both = store.fold_rows_with_pads(rhos)
        assert (both[:, :n] == store.fold_rows(rhos)).all()
        assert (both[:, n:] == o.fold_rows(pads, rows, q, q, 1, rhos)).all()
        store.free()
        cases += 1
    assert cases >= 8
    dev.ctx.set_encoder(True)


@pytest.mark.parametrize("shape", [(15, 2, 37, 280), (16, 2, 9, 280), (15, 4, 5, 40000)])
def test_rows_longer_than_one_shared_memory_transform(dev, oracle, shape):
    """The T256 / T512 profiles commit rows of 2^15 / 2^16 words (shape.rs:248-262); such a row runs as 2 or 4
    transforms of 2^14 each way.  Hiding + keyed commit: leaves, salted tree and complete opening bytes against the
    CPU; plain commit: leaves.  The third shape has q > n (pads interleave, encode_buffer.rs:56-64)."""
    o = oracle
    log_cols, ir, rows, q = shape
    n, nn = 1 << log_cols, (1 << log_cols) * ir
    tag = o.HashTag.for_profile("hashline-zk-mr1/metal-test/1")
    p = o.PcsParams(log_cols, ir, 8)
    data = rnd(700 + log_cols, rows * n)
    cpu = o.commit_zk(p, data, 18, q, o.ZkRng(77, b"long-rows"), tag)
    rng = o.ZkRng(77, b"long-rows")
    pads, salts = rng.fp_vec(rows * q), rng.salts(nn)
    got = dev.try_commit_zk_keyed(log_cols, ir, data, pads, o.coset_powers(7, nn), 18, tag.column)
    assert got is not None, dev.ctx.declines
    store, leaves = got
    assert (leaves == cpu.leaves).all()
    levels = store.merkle(salts, tag.leaf, tag.node)
    assert bytes(levels[-1]) == cpu.root and (levels == cpu.levels).all()
    cpu.mask_rows, cpu.prox_mask_row = [rows - 3, rows - 2], rows - 1
    cl = _claims(o, rows, log_cols, 1700 + log_cols)
    t1, t2 = o.Transcript(b"long-open"), o.Transcript(b"long-open")
    assert o.open_zk(cpu, cl, t1).to_bytes() == o.open_zk(cpu, cl, t2, fold=store.fold_rows_with_pads, columns=store.columns).to_bytes()
    assert t1.challenge_fp2() == t2.challenge_fp2()
    store.free()
    enc = o.encode_rows_plain(data, rows, n, nn, 18)
    store, leaves = dev.try_commit(log_cols, ir, data, 18)
    assert (leaves == o.hash_columns(enc, rows, nn)).all()
    idx = np.array([0, 1, nn - 1, nn // 2 + 3], dtype=np.uint64)
    assert (store.columns(idx) == o.gather_columns(enc, rows, nn, idx)).all()
    store.free()


def test_fold_with_sparse_dense_and_zero_vectors_in_one_call(dev, oracle):
    """An opening mixes group vectors that live on a few rows with a dense proximity vector (pcs.rs:851-891, 952-973); the
    store routes them to two kernels and must return them in the caller's order.  Also: an all-zero vector, a vector at
    the routing threshold, the plain (systematic) store."""
    o = oracle
    log_cols, ir, rows, q = 9, 4, 320, 24
    n, nn = 1 << log_cols, (1 << log_cols) * ir
    data, pads = rnd(31, rows * n), rnd(32, rows * q)
    full = np.stack([rnd2(40 + g, rows) for g in range(9)])
    rhos = np.zeros_like(full)
    rhos[0] = full[0]                       # dense
    rhos[1, 5:37] = full[1, 5:37]           # a plane's 32 rows
    rhos[2, 317:320] = full[2, 317:320]     # the mask rows at the end
    # rhos[3] stays all zero
    rhos[4, ::8] = full[4, ::8]             # exactly rows / 8 non-zero rows: still the list kernel
    rhos[5, ::7] = full[5, ::7]             # just above: the dense kernel
    rhos[6] = full[6]
    rhos[7, 100, 1] = full[7, 100, 1]       # a single imaginary word
    rhos[8, 0:40] = full[8, 0:40]
    store, _ = dev.try_commit_zk_keyed(log_cols, ir, data, pads, o.coset_powers(7, nn), 12, None)
    want = np.concatenate([o.fold_rows(data, rows, n, n, 1, rhos), o.fold_rows(pads, rows, q, q, 1, rhos)], axis=1)
    assert (store.fold_rows_with_pads(rhos) == want).all()
    assert (store.fold_rows(rhos) == want[:, :n]).all()
    store.free()
    store, _ = dev.try_commit(log_cols, ir, data, 12)
    assert (store.fold_rows(rhos) == want[:, :n]).all()
    store.free()


def _splitmix_fp(seed, n):
    out, s = [], seed
    for _ in range(n):
        s = (s + 0x9E3779B97F4A7C15) & M64
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        out.append((z ^ (z >> 31)) % P)
    return np.array(out, dtype=np.uint64)


@pytest.mark.parametrize("fast", [True, False])
def test_encode_conformance_vectors_on_the_device(dev, oracle, golden_dir, fast):
    """The 35 pinned row digests of encode_conformance_tests.rs:90-140, read back through `columns`."""
    dev.ctx.set_encoder(fast)
    g = json.load(open(os.path.join(golden_dir, "encode_vectors.json")))
    for v in g["vectors"]:
        n, q, nn, kind = int(v["n"]), int(v["q_pad"]), int(v["nn"]), v["name"].split("-", 1)[1]
        msg, pad = np.zeros(n, dtype=np.uint64), np.zeros(q, dtype=np.uint64)
        if kind == "zero_msg_seeded_pad":
            pad = _splitmix_fp(int(v["pad_seed"]), q)
        elif kind == "delta0":
            msg[0] = 1
        elif kind == "delta_last":
            msg[n - 1] = 1
        elif kind == "seeded":
            msg, pad = _splitmix_fp(int(v["msg_seed"]), n), _splitmix_fp(int(v["pad_seed"]), q)
        got = dev.try_commit_zk(int(v["log_n"]), int(v["inv_rate"]), msg, pad, oracle.coset_powers(7, nn), 18)
        assert got is not None, dev.ctx.declines
        store, _ = got
        row = np.concatenate([store.columns(np.arange(lo, min(lo + 32768, nn), dtype=np.uint64))[:, 0] for lo in range(0, nn, 32768)])
        store.free()
        assert hashlib.sha256(row.tobytes()).hexdigest() == v["encoded_sha256"], v["name"]
    dev.ctx.set_encoder(True)


def test_l5_whole_tagged_openings_on_the_device(dev, oracle, golden_dir):
    """The three seeded openings of the L5 corpus (lean_l5_export.rs:342-427) with the device as the store."""
    o = oracle
    cases = {"rungg": ("hashline-zk-mr1/private-block-rung-g-t24-dev/1", 4, 4, 12, 31), "m125": ("hashline-zk-mr1/private-block-m125/1", 5, 2, 20, 32),
             "legacy": (None, 4, 4, 12, 33)}
    recs = [l.rstrip("\n").split(" ") for l in open(os.path.join(golden_dir, "l5_corpus.txt")) if l.startswith("PCS")]
    heads = [r for r in recs if r[0] == "PCS"]
    ends = [r for r in recs if r[0] == "PCSEND"]
    for head, end in zip(heads, ends):
        profile, log_cols, ir, q, seed = cases[head[1]]
        tag = o.HashTag.for_profile(profile) if profile else o.HashTag.legacy()
        p = o.PcsParams(log_cols, ir, q)
        n, nn, rows = p.cols, p.enc_cols, 3
        rng = o.ZkRng(seed, b"lean-l5 pcs corpus")
        d = np.array([o.fp_from_i64(((i * 37) % 256) - 128) for i in range(rows * n)], dtype=np.uint64)
        for rr in (1, 2):
            for j in range(n):
                d[rr * n + j] = rng.fp()
        pads, salts = rng.fp_vec(rows * q), rng.salts(nn)
        store, leaves = dev.try_commit_zk_keyed(log_cols, ir, d, pads, o.coset_powers(7, nn), log_cols + 4, tag.column)
        levels = store.merkle(salts, tag.leaf, tag.node)
        assert bytes(levels[-1]).hex() == head[3]
        cmz = o.CommittedZk(p, rows, q, d, pads, salts, None, leaves, levels, [1], 2)
        pt = np.array([[3000 + i * 7 + 3, 3 + i * 11 + 5] for i in range(log_cols)], dtype=np.uint64)
        e = (99991, 7)
        one_e = o.fp2_sub((1, 0), e)
        vp, vr = o.eval_mle_base(d[0:n], pt), o.eval_mle_base(d[n:2 * n], pt)
        claims = [o.ZClaim([o.ZPart(0, log_cols, one_e, pt), o.ZPart(n, log_cols, e, pt)], o.fp2_add(o.fp2_mul(one_e, vp), o.fp2_mul(e, vr)))]
        tr = o.Transcript(bytes.fromhex(head[2]), tag.transcript)
        tr.absorb(b"root", bytes(levels[-1]))
        o.open_zk(cmz, claims, tr, fold=store.fold_rows_with_pads, columns=store.columns)
        assert tr.state.hex() == end[1], head[1]
        store.free()


def test_config1_commit_micro_workload(dev, oracle):
    """4096 rows x 2^10 -> 2^12, Q = 256, legacy and keyed: leaves, salted root (bit-exact with the CPU)."""
    o = oracle
    log_cols, ir, q, rows = 10, 4, 256, 4096
    n, nn = 1 << log_cols, (1 << log_cols) * ir
    data = _splitmix_vec(0xB2000001, rows * n)
    rng = o.ZkRng(0xB2000001, b"b200-cfg1")
    data[(rows - 3) * n:] = rng.fp_vec(3 * n)  # the hiding rows (protocol.rs:2371)
    for tag in (o.HashTag.legacy(), o.HashTag.for_profile("hashline-zk-mr1/b200-bench/1")):
        r2 = o.ZkRng(0xB2000001, b"b200-cfg1-commit")
        cpu = o.commit_zk(o.PcsParams(log_cols, ir, q), data, 12, q, r2, tag)
        r3 = o.ZkRng(0xB2000001, b"b200-cfg1-commit")
        pads, salts = r3.fp_vec(rows * q), r3.salts(nn)
        store, leaves = dev.try_commit_zk_keyed(log_cols, ir, data, pads, o.coset_powers(7, nn), 12, tag.column)
        assert (leaves == cpu.leaves).all()
        assert bytes(store.merkle(salts, tag.leaf, tag.node)[-1]) == cpu.root
        store.free()


def _splitmix_vec(seed, n):
    i = np.arange(1, n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + i * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z % np.uint64(P)


def test_block_size_commit_properties(dev, oracle):
    """The 8B block's `A` shape (2,504 x 2^14 -> 2^15, Q = 280, keyed) is too large to re-encode whole on
    the CPU inside a test, so it is checked through size-independent properties: sampled rows equal the
    oracle's encoding, sampled column leaves equal the oracle's hash of the gathered column, the tree over
    the device leaves equals the oracle's tree, and the fold is linear in rho."""
    o = oracle
    log_cols, ir, q, rows = 14, 2, 280, 2504
    n, nn = 1 << log_cols, (1 << log_cols) * ir
    tag = o.HashTag.for_profile("hashline-zk-mr1/b200-bench/1")
    data = _splitmix_vec(0xB2000005, rows * n)
    pads = _splitmix_vec(0xB2000006, rows * q)
    pows = o.coset_powers(7, nn)
    store, leaves = dev.try_commit_zk_keyed(log_cols, ir, data, pads, pows, 15, tag.column)
    cols = np.array([0, 1, 2, 31, 32, 4097, nn // 2, nn - 2, nn - 1, 12345], dtype=np.uint64)
    got_cols = store.columns(cols)
    for r in (0, 1, 777, rows - 1):
        want = o.encode_row_zk(data[r * n:(r + 1) * n], pads[r * q:(r + 1) * q], pows, 15)
        assert (got_cols[:, r] == want[cols.astype(np.int64)]).all(), f"row {r}"
    for c, j in enumerate(cols):
        assert bytes(leaves[int(j)]) == o.blake3(got_cols[c].tobytes(), tag.column), f"leaf {j}"
    salts = np.frombuffer(o.blake3(b"salts", None, nn * 32), dtype=np.uint8).reshape(nn, 32)
    lv = store.merkle(salts, tag.leaf, tag.node)
    assert (lv == o.merkle_build(o.salt_leaves(leaves, salts, tag.leaf), tag.node)).all()
    rho = np.stack([rnd2(1, rows), rnd2(2, rows)])
    rho_sum = np.array([[o.fp_add(int(a[0]), int(b[0])), o.fp_add(int(a[1]), int(b[1]))] for a, b in zip(rho[0], rho[1])], dtype=np.uint64)
    f = store.fold_rows_with_pads(np.concatenate([rho, rho_sum[None]]))
    s01 = (f[0].astype(object) + f[1].astype(object)) % P
    assert (s01 == f[2].astype(object)).all()
    want0 = o.fold_rows(data, rows, n, n, 1, rho[:1])
    assert (f[0, :n] == want0[0]).all()
    store.free()


def test_verifier_encodes_the_clear_vectors_through_the_commit_entry(dev, oracle):
    """verify_zk_tagged (pcs.rs:1290-1302) encodes every clear vector of an opening (group vectors and the proximity vector, real and
    imaginary parts apart) with encode_row_zk(v[..n], v[n..]) and reads the encodings at the opened indices: on the device that is
    a hiding commitment whose data rows are the vectors' heads and whose pad rows are their tails, followed by the store's column
    gather; the column hash that comes with it is not used."""
    o = oracle
    log_cols, ir, q, nvec, nidx = 10, 2, 40, 7, 33
    n, nn = 1 << log_cols, (1 << log_cols) * ir
    vecs = o.ZkRng(71, b"verify-vecs").fp2_vec(nvec * (n + q)).reshape(nvec, n + q, 2)
    idx = o.ZkRng(72, b"verify-idx").fp_vec(nidx) % np.uint64(nn)
    pows = o.coset_powers(7, nn)
    rows = np.concatenate([vecs[:, :, 0], vecs[:, :, 1]])            # 2 nvec rows of n + q words: re parts, then im parts
    heads, tails = np.ascontiguousarray(rows[:, :n]), np.ascontiguousarray(rows[:, n:])
    got = dev.try_commit_zk_keyed(log_cols, ir, heads.reshape(-1), tails.reshape(-1), pows, log_cols + 1, None)
    assert got is not None
    store, _ = got
    cols = store.columns(idx)                                        # (nidx, 2 nvec)
    for g in range(nvec):
        ere = o.encode_row_zk(heads[g], tails[g], pows, log_cols + 1)
        eim = o.encode_row_zk(heads[nvec + g], tails[nvec + g], pows, log_cols + 1)
        assert (cols[:, g] == ere[idx.astype(np.int64)]).all() and (cols[:, nvec + g] == eim[idx.astype(np.int64)]).all()
    store.free()


def test_rows_from_pageable_and_from_page_locked_memory_give_the_same_commitment(dev, oracle):
    """A large commitment is uploaded in pieces; rows in ordinary pageable memory go through the context's staging buffers (filled by
    host threads), rows in page-locked memory are copied directly, rows already on the device are not copied: one commitment."""
    import torch

    o = oracle
    log_cols, ir, q, rows = 14, 2, 280, 640
    n, nn = 1 << log_cols, (1 << log_cols) * ir
    data = rnd(4242, rows * n)
    pads, pows = rnd(4243, rows * q), o.coset_powers(7, nn)
    a = dev.try_commit_zk_keyed(log_cols, ir, data, pads, pows, log_cols + 1, None)
    pinned = torch.from_numpy(data.view(np.int64)).pin_memory().numpy().view(np.uint64)
    b = dev.try_commit_zk_keyed(log_cols, ir, pinned, pads, pows, log_cols + 1, None)
    assert a is not None and b is not None and (a[1] == b[1]).all()
    d_data, d_pads, d_pows = (torch.from_numpy(x.view(np.int64)).cuda() for x in (data, pads, pows))
    d_leaves = torch.empty(nn * 32, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    st = dev.commit_zk_dev(log_cols, ir, d_data.data_ptr(), rows, d_pads.data_ptr(), q, d_pows.data_ptr(), None, d_leaves.data_ptr())
    dev.ctx.sync()
    assert (d_leaves.cpu().numpy().reshape(nn, 32) == a[1]).all()
    # and the rows themselves: three sampled rows against the CPU encoder, through the opened columns of the first commitment
    idx = np.arange(0, nn, 997, dtype=np.uint64)
    cols = a[0].columns(idx)
    for r in (0, 255, 639):
        enc = o.encode_row_zk(data[r * n:(r + 1) * n], pads[r * q:(r + 1) * q], pows, log_cols + 1)
        assert (cols[:, r] == enc[idx.astype(np.int64)]).all()
    for x in (a[0], b[0], st):
        x.free()
