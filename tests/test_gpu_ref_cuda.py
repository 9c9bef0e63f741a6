"""This repository's kernels == the reference's OWN CUDA kernels == the CPU oracle, on the same inputs.

The reference's hashline/src/gpu/kernels.cu is compiled unchanged for sm_100a (oracle/ref_cuda.py, a checker like the rest of
oracle/) and launched with the launch shapes of hashline/src/gpu/cuda.rs.  Where the CPU oracle is the builder's restatement
of the Rust, these kernels are reference code running here: agreement with them pins the parts of the oracle that no golden
file covers (LogUp helper columns, eq tables, the sumcheck fold) and re-pins the encode, the column hash and the opening fold.
Integer and byte work: bit-exact."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
P = 0xFFFFFFFF00000001
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def ref():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_cuda

    if not ref_cuda.available():
        pytest.skip("oracle/_ref/kernels.cubin is not built: the reference checkout was not present at build time")
    return ref_cuda.RefCuda(max_log=16)


@pytest.fixture(scope="module")
def dev():
    from intelligenceregulation_b200 import backend

    d = backend.B200Backend(device=0)
    yield d
    d.ctx.close()


def _words(seed, n):
    return np.random.default_rng(seed).integers(0, P, size=n, dtype=np.uint64)


# (log_n, inv_rate, q, rows): below and above the reference's 2^12 tile, ragged row counts, rate 1/2 and 1/4, q > n / 2
SHAPES = [(10, 4, 64, 130), (12, 2, 280, 33), (13, 2, 40, 7), (14, 2, 280, 19), (9, 4, 300, 257), (11, 2, 1, 5)]


@pytest.mark.parametrize("shape", SHAPES)
def test_hiding_encode_and_column_hash_equal_the_reference_kernels(ref, dev, oracle, shape):
    import torch

    log_n, ir, q, rows = shape
    n, nn = 1 << log_n, ir << log_n
    log_nn = nn.bit_length() - 1
    data, pads, pows = _words(1, rows * n), _words(2, rows * q), oracle.coset_powers(7, nn)
    key = bytes(range(32))
    d_data, d_pads, d_pows = ref.to_dev(data), ref.to_dev(pads), ref.to_dev(pows)
    enc_ref = ref.encode_zk(d_data, d_pads, d_pows, rows, log_n, log_nn, q)
    for k in (None, key):
        leaves_ref = ref.hash_cols(enc_ref, rows, nn, k)
        st = dev.commit_zk_dev(log_n, ir, d_data.data_ptr(), rows, d_pads.data_ptr(), q, d_pows.data_ptr(), k)
        dev.ctx.sync()
        mine = ref.from_ptr(st.encoded_dev(), rows * nn)
        assert torch.equal(mine, enc_ref), "encoding differs from the reference's kernels"
        leaves = ref.from_ptr(st.leaves_dev(), nn * 4)
        assert torch.equal(leaves.view(torch.int32), leaves_ref), "column leaves differ from the reference's kernel"
        st.free()
    # and both equal the CPU oracle
    want = oracle.encode_rows_zk(data, rows, n, pads, q, pows, log_nn)
    assert (ref.to_host_u64(enc_ref) == want.reshape(-1)).all()
    assert (leaves_ref.cpu().numpy().view(np.uint8).reshape(nn, 32) == oracle.hash_columns(want, rows, nn, key)).all()


@pytest.mark.parametrize("shape", [(10, 4, 130), (13, 2, 9), (14, 2, 21), (12, 4, 40)])
def test_systematic_encode_equals_the_reference_kernels(ref, dev, oracle, shape):
    import torch

    log_n, ir, rows = shape
    n, nn = 1 << log_n, ir << log_n
    log_nn = nn.bit_length() - 1
    data = _words(3, rows * n)
    enc_ref = ref.encode_plain(ref.to_dev(data), rows, log_n, log_nn)
    store, leaves = dev.try_commit(log_n, ir, data, log_nn)
    dev.ctx.sync()
    assert torch.equal(ref.from_ptr(store.encoded_dev(), rows * nn), enc_ref)
    assert (ref.hash_cols(enc_ref, rows, nn, None).cpu().numpy().view(np.uint8).reshape(nn, 32) == leaves).all()
    assert (ref.to_host_u64(enc_ref) == oracle.encode_rows_plain(data, rows, n, nn, log_nn).reshape(-1)).all()
    store.free()


@pytest.mark.parametrize("shape", [(10, 130, 4), (12, 57, 3), (9, 300, 1)])
def test_opening_fold_equals_the_reference_kernel(ref, dev, oracle, shape):
    log_n, rows, k = shape
    n = 1 << log_n
    data = _words(4, rows * n)
    rhos = _words(5, k * rows * 2).reshape(k, rows, 2)
    got_ref = ref.to_host_u64(ref.fold_rows(ref.to_dev(data), ref.to_dev(rhos.reshape(-1)), rows, n, k)).reshape(k, n, 2)
    store, _ = dev.try_commit(log_n, 2, data, log_n + 1)
    assert (store.fold_rows(rhos) == got_ref).all()
    assert (oracle.fold_rows(data, rows, n, n, 1, rhos) == got_ref).all()
    store.free()


def test_sumcheck_fold_equals_the_reference_kernel(ref, dev, oracle):
    """Every fold of a 4-table sumcheck through both: the reference's `k_sc_fold` on its own copy of the tables, this
    repository's evaluator on its own; the tables after all folds (the finals) are equal, and so is every intermediate
    round message computed by the oracle from the reference-folded tables."""
    from intelligenceregulation_b200 import backend

    nvars, k = 11, 4
    L = 1 << nvars
    tables = _words(6, k * L * 2).reshape(k, L, 2)
    t_ref = ref.to_dev(tables.reshape(-1))
    ev = backend.B200Rounds(dev.ctx, backend.POLY_ZC, tables, 3)
    tr = oracle.Transcript(b"ref-fold")
    half = L // 2
    for j in range(nvars):
        cur = ref.to_host_u64(t_ref).reshape(k, L, 2)[:, : 2 * half]
        want = oracle.sc_round(oracle.POLY_ZC, np.ascontiguousarray(cur), 3)
        got = ev.round(j)
        assert (got == want).all(), j
        tr.absorb_fp2(b"sc-round", got)
        r = tr.challenge_fp2()
        ev.fold(r)
        ref.sc_fold(t_ref, k, half, L, r)
        half //= 2
    fin_ref = ref.to_host_u64(t_ref).reshape(k, L, 2)[:, 0]
    assert (ev.finals() == fin_ref).all()
    ev.free()


@pytest.mark.parametrize("nv", [1, 7, 10, 11, 16, 19])
def test_eq_table_equals_the_reference_kernels(ref, dev, oracle, nv):
    from intelligenceregulation_b200 import backend

    point = oracle.ZkRng(800 + nv, b"ref-eq").fp2_vec(nv)
    got_ref = ref.to_host_u64(ref.eq_table(point)).reshape(-1, 2)
    t = backend.B200Tables(dev.ctx, 1, nv)
    t.plan_eq(0, point, 0)
    t.flush()
    assert (t.read(0) == got_ref).all()
    assert (oracle.eq_table_msb(point) == got_ref).all()
    t.free()


def test_logup_helper_columns_equal_the_reference_kernel(ref, dev, oracle):
    """`k_helper` (kernels.cu:996-1040): h = 1 / (alpha - (v1 + beta w + c1)) + 1 / (alpha - (v2 + c2)) over base-field columns
    of the resident `A` data.  Without the w column this is the table-indexed pair helper of protocol.rs:1186-1216 with
    c1, c2 the two tags: this repository's `lookup_helpers_dev` (inverse tables + lookups) and the oracle's restatement must
    write the same planes, for in-table words, words beyond the table (direct inversion) and negative words.  With the w
    column it is the query form `idx + beta out + tag` of the single-term helper, checked through the oracle's arithmetic."""
    import torch

    o = oracle
    n = 5000  # not a multiple of the kernel's 8-element chunks
    rng = np.random.default_rng(7)
    a_small = rng.integers(0, 256, size=n).astype(np.int64)
    b_mixed = rng.integers(-300, 70000, size=n).astype(np.int64)  # below zero and beyond a 2^16 table
    alpha, beta = (0x1234567890ABCDEF % P, 0x0FEDCBA987654321 % P), (77777777777, 88888888888)
    g_a, g_b = (133 * 5 % P, 133 * 7 % P), (129 * 5 % P, 129 * 7 % P)
    to_fp = lambda v: np.where(v >= 0, v.astype(np.uint64), (v + (1 << 32)).astype(np.uint64) + np.uint64(P - (1 << 32)))  # noqa: E731
    a_dev = ref.to_dev(np.concatenate([to_fp(a_small), to_fp(b_mixed)]))
    h_ref = torch.zeros(2 * n, dtype=torch.int64, device="cuda")
    ref.helper(a_dev, 0, -1, n, n, alpha, beta, g_a, g_b, h_ref, 0, n)
    re_ref, im_ref = ref.to_host_u64(h_ref[:n]), ref.to_host_u64(h_ref[n:])
    # the oracle
    tab_a, tab_b = o.lookup_inverse_table(alpha, g_a, 256), o.lookup_inverse_table(alpha, g_b, 1 << 16)
    got = o.lookup_helpers(a_small, tab_a, g_a, alpha, b_mixed, tab_b, g_b)
    assert got is not None and (got[0] == re_ref).all() and (got[1] == im_ref).all()
    # this repository's kernels
    d_ta = torch.empty(2 * 256, dtype=torch.int64, device="cuda")
    d_tb = torch.empty(2 << 16, dtype=torch.int64, device="cuda")
    d_a, d_b = torch.from_numpy(a_small).cuda(), torch.from_numpy(b_mixed).cuda()
    d_re, d_im = torch.empty(n, dtype=torch.int64, device="cuda"), torch.empty(n, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    dev.ctx.lookup_inverse_table(alpha, g_a, 8, d_ta.data_ptr())
    dev.ctx.lookup_inverse_table(alpha, g_b, 16, d_tb.data_ptr())
    dev.ctx.lookup_helpers_dev(d_a.data_ptr(), d_ta.data_ptr(), 8, g_a, alpha, n, d_re.data_ptr(), d_im.data_ptr(), d_b.data_ptr(), d_tb.data_ptr(), 16, g_b)
    dev.ctx.sync()
    assert (ref.to_host_u64(d_re) == re_ref).all() and (ref.to_host_u64(d_im) == im_ref).all()
    # with the w column: h - 1 / (alpha - (v2 + c2)) is the single-term query helper 1 / (alpha - (idx + beta out + tag))
    idx, outv = rng.integers(0, 1 << 16, size=n).astype(np.int32), rng.integers(-32768, 32768, size=n).astype(np.int32)
    a2 = ref.to_dev(np.concatenate([to_fp(idx.astype(np.int64)), to_fp(outv.astype(np.int64)), to_fp(a_small)]))
    h2 = torch.zeros(2 * n, dtype=torch.int64, device="cuda")
    ref.helper(a2, 0, n, 2 * n, n, alpha, beta, g_a, g_b, h2, 0, n)
    single = o.logup_helpers(idx, outv, alpha, beta, g_a)
    mine = dev.ctx.logup_helpers(idx, outv, alpha, beta, g_a)
    assert (mine == single).all()
    re2, im2 = ref.to_host_u64(h2[:n]), ref.to_host_u64(h2[n:])
    for i in list(range(0, n, 97)) + [n - 1]:
        second = o.fp2_inv(o.fp2_sub(alpha, o.fp2_add((int(a_small[i]), 0), g_b)))
        assert o.fp2_add(tuple(map(int, single[i])), second) == (int(re2[i]), int(im2[i])), i


def test_block_shape_commitment_equals_the_reference_kernels(ref, dev, oracle):
    """The Llama-3-8B block `A` shape at full size (2,504 rows of 2^14 words to 2^15, 280 pads, keyed leaves): this
    repository's encoding and leaves against the reference's kernels, every word."""
    import torch

    log_n, ir, q, rows = 14, 2, 280, 2504
    n, nn = 1 << log_n, ir << log_n
    d_data, d_pads, d_pows = ref.to_dev(_words(11, rows * n)), ref.to_dev(_words(12, rows * q)), ref.to_dev(oracle.coset_powers(7, nn))
    key = bytes(range(7, 39))
    enc_ref = ref.encode_zk(d_data, d_pads, d_pows, rows, log_n, 15, q)
    leaves_ref = ref.hash_cols(enc_ref, rows, nn, key)
    st = dev.commit_zk_dev(log_n, ir, d_data.data_ptr(), rows, d_pads.data_ptr(), q, d_pows.data_ptr(), key)
    dev.ctx.sync()
    assert torch.equal(ref.from_ptr(st.encoded_dev(), rows * nn), enc_ref)
    assert torch.equal(ref.from_ptr(st.leaves_dev(), nn * 4).view(torch.int32), leaves_ref)
    st.free()
