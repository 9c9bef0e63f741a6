"""The matmul-claim and LogUp benchmark configurations (called config 2 and config 3 below) on the device against the CPU oracle (bit-exact).

Config 2: masked sumcheck of one integer matmul C = A B (A int8 128 x 4096, B int8 4096 x 4096): the two
weight folds, the 12-round product sumcheck under a CFS mask, one extension round, transcript end state.
Config 3: LogUp over a 2^16-entry table and 128 x 14336 queries padded to 2^21: multiplicities, helper
columns, table helpers, the value-0 identity sum h - sum h_t = 0, and both zero-check sumchecks.
Inputs are seeded synthetic data of the named shapes and distributions.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
P = 0xFFFFFFFF00000001


@pytest.fixture(scope="module")
def ctx():
    from intelligenceregulation_b200 import backend

    c = backend.Context(0)
    yield c
    c.close()


def t2(x):
    return (int(x[0]), int(x[1]))


def test_config2_masked_matmul_sumcheck(ctx, oracle):
    o = oracle
    from intelligenceregulation_b200 import backend

    g = np.random.default_rng(0xB2000002)
    A = g.integers(-128, 128, size=(128, 4096), dtype=np.int8)
    B = np.clip(np.rint(g.normal(0.0, 32.0, size=(4096, 4096))), -128, 127).astype(np.int8)
    tr = o.Transcript(b"b200-cfg2")
    r_i, r_j = tr.challenge_fp2_vec(7), tr.challenge_fp2_vec(12)
    eq_i, eq_j = o.eq_table_msb(r_i), o.eq_table_msb(r_j)
    # T0[k] = sum_i eq(r_i)[i] A[i][k]; T1[k] = sum_j eq(r_j)[j] B[k][j]   (mle.rs fold_rows_i8 / fold_cols_i8)
    T0, T1 = ctx.fold_rows_i8(A, eq_i), ctx.fold_cols_i8(B, eq_j)
    assert (T0 == o.fold_rows_i8(A, eq_i)).all()
    assert (T1 == o.fold_cols_i8(B, eq_j)).all()
    tables = np.stack([T0, T1])
    n, deg = 12, 2
    mask = o.ZkRng(0xB2000002, b"b200-cfg2").fp2_vec((n + 1) * deg + 2)  # CfsMask::random(.., 13, 2)
    cc = tr.challenge_fp2()
    assert cc != (0, 0)
    t_cpu = tr.clone()
    want = o.sc_prove(o.POLY_PROD, tables, deg, t_cpu, mask=mask, mask_c=cc, mask_vars=n + 1)
    ev = backend.B200Rounds(ctx, backend.POLY_PROD, tables, deg)
    sums, absorbed, ch, st, ctr, _ = ev.batched(n, tr.state, tr.counter, None, mask=mask, mask_vars=n + 1, mask_c=cc, recover_one=True)
    assert (sums == want.rounds).all() and (absorbed == want.masked).all() and (ch == want.challenges).all()
    finals = ev.finals()
    assert (finals == want.finals).all()
    ev.free()
    # the extension round on the finals (sumcheck.rs:302-314), masked, absorbed by both transcripts
    exts = o.ZkRng(9, b"b200-cfg2-ext").fp2_vec(2)
    t_dev = o.Transcript(b"b200-cfg2")
    t_dev._t.state[:] = list(st)
    t_dev._t.counter = ctr
    for t, f, c_ in ((t_cpu, want.finals, want.challenges), (t_dev, finals, ch)):
        sk = o.extension_round(o.POLY_PROD, f, exts, deg)
        gk = o.cfs_round(mask, n + 1, deg, n, c_)
        sk = np.array([o.fp2_add(t2(s), o.fp2_mul(cc, t2(g_))) for s, g_ in zip(sk, gk)], dtype=np.uint64)
        t.absorb_fp2(b"sc-round", sk)
        t.challenge_fp2()
    assert t_dev.state == t_cpu.state and t_dev.counter == t_cpu.counter


def test_config3_logup_batch(ctx, oracle):
    o = oracle
    from intelligenceregulation_b200 import backend

    g = np.random.default_rng(0xB2000003)
    table_len = 1 << 16
    x = (np.arange(table_len) - 32768) / 4096.0
    table_out = np.clip(np.rint(x / (1.0 + np.exp(-x)) * 4096.0), -32768, 32767).astype(np.int32)  # quantised SiLU, monotone enough, int16 range
    qv = np.clip(np.rint(g.normal(0.0, 4096.0, size=(128, 14336))), -32768, 32767).astype(np.int64) + 32768
    idx = np.full((128, 16384), 32768, dtype=np.int32)  # padding looks up the entry of value 0 (accuracy_act.rs:105-111)
    idx[:, :14336] = qv
    idx = idx.reshape(-1)
    outv = table_out[idx]
    tr = o.Transcript(b"b200-cfg3")
    alpha, beta, gamma = tr.challenge_fp2(), tr.challenge_fp2(), tr.challenge_fp2()
    tag = o.fp2_mul_base(gamma, 216)  # TAG_RANGE0 + 16 (range16.rs:31-36)

    mult = ctx.logup_histogram(idx, table_len)
    assert (mult == o.logup_histogram(idx, table_len)).all() and int(mult.sum()) == idx.size
    h = ctx.logup_helpers(idx, outv, alpha, beta, tag)
    assert (h == o.logup_helpers(idx, outv, alpha, beta, tag)).all()
    ht = ctx.logup_helpers(None, table_out, alpha, beta, tag, mult=mult)
    assert (ht == o.logup_table_helper(table_out, mult, alpha, beta, tag)).all()
    assert o.fp2_sub(o.fp2_sum(h), o.fp2_sum(ht)) == (0, 0)  # the LogUp identity (protocol.rs:171-189)

    # zero denominators refuse the attempt and nothing else (protocol.rs:1005-1006)
    q0 = o.logup_query_values(idx[:16], outv[:16], beta, tag)
    with pytest.raises(backend.DeviceError) as e:
        ctx.logup_helpers(idx[:16], outv[:16], t2(q0[5]), beta, tag)
    assert e.value.code == -6

    # query-side zero-check eq(tau) (h (alpha - q) - 1), 21 variables, degree 3, masked, one device batch
    for name, poly, n, hh, qq, extra in (
        ("query", backend.POLY_LOGUP_Q, 21, h, o.logup_query_values(idx, outv, beta, tag), None),
        ("table", backend.POLY_LOGUP_T, 16, ht, o.logup_query_values(None, table_out, beta, tag), mult),
    ):
        tau = tr.challenge_fp2_vec(n)
        tabs = [o.eq_table_msb(tau), hh, qq]
        if extra is not None:
            tabs.append(np.stack([extra, np.zeros_like(extra)], axis=1))
        tables = np.stack(tabs)
        mask = o.ZkRng(n, b"b200-cfg3").fp2_vec((n + 1) * 3 + 2)
        cc = tr.challenge_fp2()
        coefs = np.array([alpha], dtype=np.uint64)
        t_cpu = tr.clone()
        want = o.sc_prove(poly, tables, 3, t_cpu, coefs=coefs, mask=mask, mask_c=cc, mask_vars=n + 1, recover_one=True, claim=(0, 0))
        ev = backend.B200Rounds(ctx, poly, tables, 3, coefs)
        sums, absorbed, ch, st, ctr, _ = ev.batched(n, tr.state, tr.counter, None, mask=mask, mask_vars=n + 1, mask_c=cc, recover_one=True, claim=(0, 0))
        assert (sums == want.rounds).all(), name
        assert (absorbed == want.masked).all() and (ch == want.challenges).all()
        assert st == t_cpu.state and ctr == t_cpu.counter
        assert (ev.finals() == want.finals).all()
        # a zero-check's round polynomial sums to zero at every round start: s(0) + s(1) = running claim, first claim 0
        assert o.fp2_add(t2(sums[0][0]), t2(sums[0][1])) == (0, 0)
        ev.free()
        tr = t_cpu
