"""A slot's tables built on the device == the reference's host builders (oracle restatement of
private_block/argument.rs:386-660), word for word, and a sumcheck run over device-built tables == the same run over
host-built ones.  Mirrors the reference's own gate for its device builders ("every word of every table of every slot
compared with the host builders", gpu/metal.rs A12 notes).  Field work: bit-exact."""
import numpy as np
import pytest

import tables_util as T

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from intelligenceregulation_b200 import backend

    d = backend.B200Backend(device=0)
    yield d
    d.ctx.close()


@pytest.fixture(scope="module")
def committed(dev):
    """512 rows x 2^10 words resident on the device behind a commitment: the rows a plane table reads"""
    data = np.random.default_rng(99).integers(0, T.P, size=512 << 10, dtype=np.uint64)
    store, _ = dev.try_commit(10, 2, data, 12)
    yield store, data
    store.free()


PLANES = [  # seed, n_vars, fixed, unused, slices
    (11, 16, 0, 0, 1), (12, 16, 3, 0, 1), (13, 12, 7, 0, 1), (14, 14, 2, 3, 1), (15, 15, 0, 0, 3), (16, 13, 4, 2, 2), (17, 17, 2, 0, 1), (18, 3, 0, 1, 1),
]


@pytest.mark.parametrize("case", PLANES)
def test_plane_table_on_the_device_equals_the_host_builder(dev, oracle, committed, case):
    from intelligenceregulation_b200 import backend

    store, data = committed
    seed, n_vars, n_fixed, n_unused, ns = case
    coords, slices = T.random_plane(seed, n_vars, n_fixed, n_unused, ns, data.size)
    want = oracle.priv_table(coords, slices, data, n_vars)
    t = backend.B200Tables(dev.ctx, 2, n_vars)
    t.plan_plane(1, store, coords, slices)
    t.flush()
    assert (t.read(1) == want).all()
    t.free()


@pytest.mark.parametrize("case", [(16, 0, 16), (18, 3, 11), (12, 12, 0), (10, 0, 1), (15, 4, 7)])
def test_eq_cube_on_the_device(dev, oracle, case):
    from intelligenceregulation_b200 import backend

    n_vars, start, p = case
    point = oracle.ZkRng(7000 + n_vars + p, b"eq").fp2_vec(max(p, 1))[:p]
    t = backend.B200Tables(dev.ctx, 1, n_vars)
    t.plan_eq(0, point, start)
    t.flush()
    assert (t.read(0) == oracle.eq_cube(point, n_vars, start)).all()
    t.free()


def test_sumcheck_over_device_built_tables(dev, oracle, committed):
    """eq(tau) * (plane_a * plane_b - public): tables 0-2 planned on the device, table 3 put by the host; the masked
    batch equals the oracle's run over the host-built tables."""
    from intelligenceregulation_b200 import backend

    o = oracle
    store, data = committed
    n = 15
    tau = o.ZkRng(5, b"tau").fp2_vec(n)
    ca, sa = T.random_plane(31, n, 3, 0, 1, data.size)
    cb, sb = T.random_plane(32, n, 0, 2, 2, data.size)
    pub = o.ZkRng(6, b"pub").fp2_vec(1 << n)
    host = np.stack([o.eq_cube(tau, n, 0), o.priv_table(ca, sa, data, n), o.priv_table(cb, sb, data, n), pub])
    t = backend.B200Tables(dev.ctx, 4, n)
    t.plan_eq(0, tau, 0)
    t.plan_plane(1, store, ca, sa)
    t.plan_plane(2, store, cb, sb)
    t.put(3, pub)
    mask = o.ZkRng(8, b"mask").fp2_vec((n + 1) * 3 + 2)
    tr = o.Transcript(b"tables")
    cc = tr.challenge_fp2()
    t_cpu = tr.clone()
    want = o.sc_prove(o.POLY_ZC, host, 3, t_cpu, mask=mask, mask_c=cc, mask_vars=n + 1)
    ev = backend.B200Rounds(dev.ctx, backend.POLY_ZC, t, 3)
    claim0 = o.fp2_add(tuple(map(int, want.rounds[0][0])), tuple(map(int, want.rounds[0][1])))
    sums, absorbed, ch, st, ctr, _ = ev.batched(n, tr.state, tr.counter, None, mask=mask, mask_vars=n + 1, mask_c=cc, recover_one=True, claim=claim0)
    assert (sums == want.rounds).all() and (absorbed == want.masked).all() and (ch == want.challenges).all()
    assert st == t_cpu.state and (ev.finals() == want.finals).all()
    ev.free()


def test_refusals(dev, oracle, committed):
    from intelligenceregulation_b200 import backend

    store, data = committed
    n = 10
    coords, slices = T.random_plane(41, n, 0, 0, 1, data.size)
    # a slice that reaches past the committed rows is refused before any launch
    t = backend.B200Tables(dev.ctx, 1, n)
    launches = dev.ctx.stats()["kernel_launches"]
    with pytest.raises(backend.DeviceError):
        t.plan_plane(0, store, coords, [(data.size - 5, (1, 0))])
    assert dev.ctx.stats()["kernel_launches"] == launches
    # a table declared base-valued that is not: refused at flush, and a round evaluator is not made from it
    t.plan_plane(0, store, coords, [(0, (3, 9))], base_check=True)
    with pytest.raises(backend.DeviceError):
        t.flush()
    with pytest.raises(backend.DeviceError):
        backend.B200Rounds(dev.ctx, backend.POLY_PROD, t, 1)
    t.free()
    # declared base-valued and base-valued: accepted
    t = backend.B200Tables(dev.ctx, 1, n)
    t.plan_plane(0, store, coords, slices, base_check=True)
    t.flush()
    assert (t.read(0)[:, 1] == 0).all()
    t.free()
    # an eq point that does not fit the cube (argument.rs:604-607)
    t = backend.B200Tables(dev.ctx, 1, 4)
    with pytest.raises(backend.DeviceError):
        t.plan_eq(0, oracle.ZkRng(1, b"e").fp2_vec(3), 2)
    t.free()


def test_a_planned_plane_whose_commitment_was_freed_is_refused_not_launched(dev, oracle):
    """The eq and plane calls only plan a table; the launch comes when the set is flushed.  A commitment freed in between is found
    on the host: the flush is refused, nothing is launched over the freed rows, and the set takes new plans afterwards."""
    from intelligenceregulation_b200 import backend

    data = np.random.default_rng(7).integers(0, T.P, size=64 << 8, dtype=np.uint64)
    store, _ = dev.try_commit(8, 2, data, 10)
    coords, slices = T.random_plane(43, 10, 0, 0, 1, data.size)
    t = backend.B200Tables(dev.ctx, 2, 10)
    t.plan_plane(0, store, coords, slices)
    point = oracle.ZkRng(2, b"e").fp2_vec(10)
    t.plan_eq(1, point, 0)
    store.free()
    launches = dev.ctx.stats()["kernel_launches"]
    with pytest.raises(backend.DeviceError):
        t.flush()
    assert dev.ctx.stats()["kernel_launches"] == launches
    # the refused plan is gone: the set builds what is planned next
    store2, _ = dev.try_commit(8, 2, data, 10)
    t.plan_plane(0, store2, coords, slices)
    t.plan_eq(1, point, 0)
    t.flush()
    assert (t.read(0) == oracle.priv_table(coords, slices, data, 10)).all()
    assert (t.read(1) == oracle.eq_cube(point, 10, 0)).all()
    t.free()
    store2.free()


def test_page_locked_inputs_may_be_overwritten_when_the_call_returns(dev, oracle):
    """`tables_put`, `tables_eq` and `tables_plane` return before their copies run.  From page-locked caller memory such a
    copy reads its source when the DMA engine gets to it, so the library must have taken the bytes by then: every input
    here lives in page-locked memory and is overwritten as soon as its call returns; the tables must hold the values that
    were passed.  A large table (copied in place and waited for) and many small ones (bounced through the context's own
    page-locked area, which wraps several times) are both covered."""
    import torch
    from intelligenceregulation_b200 import backend

    def pinned(a):
        t = torch.empty(a.size, dtype=torch.int64, pin_memory=True)
        v = t.numpy().view(np.uint64).reshape(a.shape)
        v[...] = a
        return t, v

    rng = oracle.ZkRng(4242, b"pinned")
    # one large table after a long kernel, so that the copy is still queued when the call returns
    n_big = 20
    big = rng.fp2_vec(1 << n_big)
    keep, view = pinned(big)
    t = backend.B200Tables(dev.ctx, 2, n_big)
    t.plan_eq(0, rng.fp2_vec(n_big), 0)
    t.put(1, view)
    view[...] = 0
    t.flush()
    assert (t.read(1) == big).all()
    t.free()
    # many small ones: 24 KiB each through the 4 MiB bounce area, 600 calls = 3.5 wraps; eq halves the same way
    n_small, k = 9, 60
    for rep in range(10):
        want = [rng.fp2_vec(1 << n_small) for _ in range(k)]
        t = backend.B200Tables(dev.ctx, k + 1, n_small)
        keep, view = pinned(want[0])
        point = rng.fp2_vec(n_small)
        p_lo = n_small // 2
        hi, lo = backend.eq_table_msb(point[: n_small - p_lo]), backend.eq_table_msb(point[n_small - p_lo:])
        (kh, vh), (kl, vl) = pinned(hi), pinned(lo)
        dev.ctx.check(dev.ctx.lib.hl_b200_tables_eq(t.h, k, 0, n_small, backend._ptr(vh), backend._ptr(vl), 0))
        vh[...] = 0
        vl[...] = 0
        for i in range(k):
            view[...] = want[i]
            t.put(i, view)
            view[...] = 0xDEAD
        t.flush()
        for i in range(k):
            assert (t.read(i) == want[i]).all(), (rep, i)
        assert (t.read(k) == oracle.eq_cube(point, n_small, 0)).all()
        t.free()
