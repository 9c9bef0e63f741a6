"""The hiding commitment from narrow witness rows (`hl_b200_commit_zk_packed`) == the commitment of the widened matrix: leaves,
salted tree, opened columns and row combinations (which read the widened rows the encoder left resident), byte for byte, on the
reference's commit shapes, on rows shorter and longer than the fused path covers, on both encoder paths, from pageable and from
page-locked memory, and at the Llama-3-8B block shape.  The widening itself is held to the reference's own kernel
(hashline/src/gpu/kernels.cu:227-236 `k_widen`).  Integer and byte work: bit-exact."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
P = 0xFFFFFFFF00000001
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def dev():
    from intelligenceregulation_b200 import backend

    d = backend.B200Backend(device=0)
    yield d
    d.ctx.close()


def to_fp(v):
    return np.where(v >= 0, v.astype(np.uint64), (v + (1 << 32)).astype(np.uint64) + np.uint64(P - (1 << 32)))


def witness(seed, rows, n):
    """rows of int8, int16, int32 and full-width words in turn, with every class's extreme values planted"""
    rng = np.random.default_rng(seed)
    out = np.empty((rows, n), dtype=np.uint64)
    for r in range(rows):
        k = (r + seed) % 4
        if k == 0:
            out[r] = to_fp(rng.integers(-128, 128, n))
            out[r, :4] = to_fp(np.array([-128, 127, -1, 0]))[: min(4, n)]
        elif k == 1:
            out[r] = to_fp(rng.integers(-32768, 32768, n))
            out[r, :4] = to_fp(np.array([-32768, 32767, 128, -129]))[: min(4, n)]
        elif k == 2:
            out[r] = to_fp(rng.integers(-(1 << 31), 1 << 31, n))
            out[r, :4] = to_fp(np.array([-(1 << 31), (1 << 31) - 1, 32768, -32769]))[: min(4, n)]
        else:
            out[r] = rng.integers(0, P, n, dtype=np.uint64)
            out[r, :4] = np.array([P - 1, 0, 1 << 31, P - (1 << 31) - 1], dtype=np.uint64)[: min(4, n)]
    return out.reshape(-1)


def same_commitment(dev, oracle, log_cols, ir, rows, q, seed, check_oracle=True):
    from intelligenceregulation_b200 import backend

    o = oracle
    n, nn = 1 << log_cols, ir << log_cols
    data = witness(seed, rows, n)
    rng = np.random.default_rng(1000 + seed)
    pads = rng.integers(0, P, rows * q, dtype=np.uint64)
    pows = o.coset_powers(7, nn)
    salts = rng.integers(0, 256, (nn, 32), dtype=np.uint8)
    tag = o.HashTag.for_profile("hashline-zk-mr1/b200-packed/1")
    packed, widths = backend.pack_rows(data, rows)
    assert rows < 4 or set(widths.tolist()) == {1, 2, 4, 8}
    wide = dev.try_commit_zk_tree(log_cols, ir, data, pads, pows, 17, tag.column, salts, tag.leaf, tag.node)
    narrow = dev.try_commit_zk_packed(log_cols, ir, packed, widths, pads, pows, 17, tag.column, salts, tag.leaf, tag.node)
    assert wide is not None and narrow is not None, dev.ctx.declines
    (st_w, leaves_w, levels_w), (st_n, leaves_n, levels_n) = wide, narrow
    assert (leaves_n == leaves_w).all() and (levels_n == levels_w).all()
    rhos = rng.integers(0, P, (3, rows, 2), dtype=np.uint64)
    rhos[1, : rows // 2] = 0
    fold_n = st_n.fold_rows_with_pads(rhos)
    assert (fold_n == st_w.fold_rows_with_pads(rhos)).all()
    idx = np.array([0, nn - 1, nn // 3, 5 % nn, 0], dtype=np.uint64)
    assert (st_n.columns(idx) == st_w.columns(idx)).all()
    if check_oracle:
        enc = o.encode_rows_zk(data, rows, n, pads, q, pows, 17)
        assert (leaves_n == o.hash_columns(enc, rows, nn, tag.column)).all()
        want = np.concatenate([o.fold_rows(data, rows, n, n, 1, rhos), o.fold_rows(pads, rows, q, q, 1, rhos)], axis=1)
        assert (fold_n == want).all()
    # without the tree: leaves only
    st2, leaves2 = dev.try_commit_zk_packed(log_cols, ir, packed, widths, pads, pows, 17, tag.column)
    assert (leaves2 == leaves_w).all()
    for s in (st_w, st_n, st2):
        s.free()


# (log_cols, inv_rate, rows, q): the reference's commit shapes that admit pads, a ragged fast-path size of every 2^8 .. 2^14,
# rows below 2^8 words (generic encoder, widening pass of its own) and above 2^14 (several shared-memory transforms)
SHAPES = [(3, 4, 4, 12), (4, 4, 5, 8), (6, 4, 8, 8), (8, 2, 127, 8), (8, 4, 128, 8), (8, 4, 129, 300), (9, 2, 33, 40), (10, 4, 300, 64),
          (11, 2, 77, 1), (12, 4, 1100, 280), (13, 2, 150, 280), (14, 2, 75, 280), (14, 2, 300, 280), (15, 2, 37, 280), (16, 2, 9, 280)]


@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("shape", SHAPES)
def test_packed_rows_commit_to_the_same_leaves_tree_and_opening(dev, oracle, shape, fast):
    if not fast and shape[0] > 14:
        pytest.skip("rows above 2^14 words always take the shared-memory transforms")
    dev.ctx.set_encoder(fast)
    try:
        same_commitment(dev, oracle, *shape, seed=sum(shape))
    finally:
        dev.ctx.set_encoder(True)


def test_block_shape_from_pageable_and_page_locked_packed_rows(dev, oracle):
    """2,504 rows of 2^14 words (the Llama-3-8B block `A` shape), int16-valued except eight full-width rows: the upload goes in
    wave-sized pieces (82 MB of narrow bytes instead of 328 MB), from pageable memory through the context's staging buffers and from
    page-locked memory directly; leaves and tree equal the wide call's."""
    import torch
    from intelligenceregulation_b200 import backend

    o = oracle
    log_cols, ir, rows, q = 14, 2, 2504, 280
    n, nn = 1 << log_cols, ir << log_cols
    rng = np.random.default_rng(5)
    data = to_fp(rng.integers(-32768, 32768, rows * n)).reshape(rows, n)
    data[::313] = rng.integers(0, P, (8, n), dtype=np.uint64)
    data = data.reshape(-1)
    pads = rng.integers(0, P, rows * q, dtype=np.uint64)
    pows, salts = o.coset_powers(7, nn), rng.integers(0, 256, (nn, 32), dtype=np.uint8)
    tag = o.HashTag.for_profile("hashline-zk-mr1/b200-packed/1")
    packed, widths = backend.pack_rows(data, rows)
    assert sorted(set(widths.tolist())) == [2, 8] and int((widths == 8).sum()) == 8
    st_w, _, levels_w = dev.try_commit_zk_tree(log_cols, ir, data, pads, pows, 15, tag.column, salts, tag.leaf, tag.node, want_leaves=False)
    h0 = dev.ctx.stats()["bytes_h2d"]
    st_p, _, levels_p = dev.try_commit_zk_packed(log_cols, ir, packed, widths, pads, pows, 15, tag.column, salts, tag.leaf, tag.node, want_leaves=False)
    sent = dev.ctx.stats()["bytes_h2d"] - h0
    assert (levels_p == levels_w).all()
    assert sent < 100e6, sent  # 82 MB of rows + pads, salts, powers, against 335 MB for the wide call
    pin = torch.empty(packed.size, dtype=torch.uint8, pin_memory=True)
    pin.numpy()[...] = packed
    st_q, _, levels_q = dev.try_commit_zk_packed(log_cols, ir, pin.numpy(), widths, pads, pows, 15, tag.column, salts, tag.leaf, tag.node, want_leaves=False)
    assert (levels_q == levels_w).all()
    rhos = rng.integers(0, P, (2, rows, 2), dtype=np.uint64)
    assert (st_q.fold_rows_with_pads(rhos) == st_w.fold_rows_with_pads(rhos)).all()
    for s in (st_w, st_p, st_q):
        s.free()


@pytest.mark.parametrize("rows", [593, 1185, 1777, 2369])
def test_piecewise_upload_at_row_counts_around_the_piece_boundaries(dev, oracle, rows):
    """The narrow upload goes in pieces of 1, 2, 3, 5, 8 waves (a wave = one row per SM), the pads of each piece and the salts with
    them.  Row counts one above a piece boundary on a 148-SM device (4 x 148 + 1, 8 x 148 + 1, ..), where the last piece is a single
    row: the packed call from page-locked and from pageable memory, the wide call, and a commitment of the same rows already on the
    device (no pieces at all) give one tree, and the pads and widened rows left resident give the same opening combination."""
    import torch

    from intelligenceregulation_b200 import backend

    o = oracle
    log_cols, ir, q = 14, 2, 280
    n, nn = 1 << log_cols, ir << log_cols
    rng = np.random.default_rng(rows)
    data = to_fp(rng.integers(-32768, 32768, rows * n)).reshape(rows, n)
    data[::97] = rng.integers(0, P, (len(range(0, rows, 97)), n), dtype=np.uint64)
    data = data.reshape(-1)
    pads = rng.integers(0, P, rows * q, dtype=np.uint64)
    pows, salts = o.coset_powers(7, nn), rng.integers(0, 256, (nn, 32), dtype=np.uint8)
    tag = o.HashTag.for_profile("hashline-zk-mr1/b200-packed/1")
    packed, widths = backend.pack_rows(data, rows)
    # resident rows: one encoder launch, no pieces
    dd, dp = torch.from_numpy(data.view(np.int64)).cuda(), torch.from_numpy(pads.view(np.int64)).cuda()
    dw, ds = torch.from_numpy(pows.view(np.int64)).cuda(), torch.from_numpy(salts).cuda()
    dl = torch.empty((2 * nn - 1) * 32, dtype=torch.uint8, device="cuda")
    st_r = dev.commit_zk_dev(log_cols, ir, dd.data_ptr(), rows, dp.data_ptr(), q, dw.data_ptr(), tag.column)
    st_r.merkle_dev(ds.data_ptr(), tag.leaf, tag.node, dl.data_ptr())
    dev.ctx.sync()
    want = dl.cpu().numpy().reshape(2 * nn - 1, 32)
    st_w, _, levels_w = dev.try_commit_zk_tree(log_cols, ir, data, pads, pows, 15, tag.column, salts, tag.leaf, tag.node, want_leaves=False)
    assert (levels_w == want).all()
    st_p, _, levels_p = dev.try_commit_zk_packed(log_cols, ir, packed, widths, pads, pows, 15, tag.column, salts, tag.leaf, tag.node, want_leaves=False)
    assert (levels_p == want).all()
    pin = torch.empty(packed.size, dtype=torch.uint8, pin_memory=True)
    pin.numpy()[...] = packed
    pin_pads = torch.from_numpy(pads.view(np.int64)).pin_memory()
    st_q, _, levels_q = dev.try_commit_zk_packed(log_cols, ir, pin.numpy(), widths, pin_pads.numpy().view(np.uint64), pows, 15, tag.column, salts, tag.leaf, tag.node,
                                                  want_leaves=False)
    assert (levels_q == want).all()
    rhos = rng.integers(0, P, (2, rows, 2), dtype=np.uint64)
    ref = st_r.fold_rows_with_pads(rhos)
    for s in (st_w, st_p, st_q):
        assert (s.fold_rows_with_pads(rhos) == ref).all()
        s.free()
    st_r.free()


def test_refusals(dev, oracle):
    from intelligenceregulation_b200 import backend

    n, rows, q = 256, 4, 8
    data = witness(1, rows, n)
    packed, widths = backend.pack_rows(data, rows)
    pads, pows = np.zeros(rows * q, dtype=np.uint64), oracle.coset_powers(7, 2 * n)
    bad = widths.copy()
    bad[1] = 3
    packed3 = np.zeros(int(bad.astype(np.int64).sum()) * n, dtype=np.uint8)
    launches = dev.ctx.stats()["kernel_launches"]
    assert dev.try_commit_zk_packed(8, 2, packed3, bad, pads, pows, 9, None) is None
    assert "width" in dev.ctx.declines[-1][1]
    assert dev.ctx.stats()["kernel_launches"] == launches


def test_widening_equals_the_reference_kernel(oracle):
    """`k_widen` of the reference, compiled for sm_100a, on the packed bytes of each width == the words that were packed."""
    import torch
    from intelligenceregulation_b200 import backend

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_cuda

    if not ref_cuda.available():
        pytest.skip("oracle/_ref/kernels.cubin is not built: the reference checkout was not present at build time")
    ref = ref_cuda.RefCuda(max_log=4)
    n = 4096
    for r, w in ((0, 1), (1, 2), (2, 4)):
        row = witness(0, 4, n).reshape(4, n)[r]
        packed, widths = backend.pack_rows(row, 1)
        assert int(widths[0]) == w
        got = ref.widen(torch.from_numpy(packed.copy()).cuda(), n, w)
        assert (ref.to_host_u64(got) == row).all()
