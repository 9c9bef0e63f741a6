"""LogUp helper columns of table-indexed lookups on the device == the CPU restatement of protocol.rs:1125-1230
(u8_denominator_inverses, helper_one, helper_pair_inverses_u8), itself checked in test_lookup_cpu.py against the
element-wise batch inversion the reference's own tests compare the table form with.  Field words: bit-exact; the refusal
falls exactly where the reference's does (a zero denominator at a value the column carries, never at an absent one)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import torch
    from intelligenceregulation_b200 import backend

    torch.cuda.set_device(0)
    d = backend.B200Backend(device=0)
    yield d
    d.ctx.close()


def _dev_table(dev, alpha, g, log_len):
    import torch

    t = torch.empty((1 << log_len) * 2, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    dev.ctx.lookup_inverse_table(alpha, g, log_len, t.data_ptr())
    return t


def _run(dev, a, ta, la, ga, alpha, b=None, tb=None, lb=0, gb=None):
    import torch

    d_a = torch.from_numpy(np.ascontiguousarray(a, np.int64)).cuda()
    d_b = torch.from_numpy(np.ascontiguousarray(b, np.int64)).cuda() if b is not None else None
    re = torch.zeros(len(a), dtype=torch.int64, device="cuda")
    im = torch.zeros(len(a), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    dev.ctx.lookup_helpers_dev(d_a.data_ptr(), ta.data_ptr(), la, ga, alpha, len(a), re.data_ptr(), im.data_ptr(),
                               d_b=d_b.data_ptr() if b is not None else 0, d_table_b=tb.data_ptr() if b is not None else 0, log_b=lb, g_b=gb)
    return re.cpu().numpy().view(np.uint64), im.cpu().numpy().view(np.uint64)


@pytest.mark.parametrize("log_len", [0, 3, 8, 16, 19])
def test_inverse_table(dev, oracle, log_len):
    import torch

    r = oracle.ZkRng(40 + log_len, b"lookup")
    alpha, g = r.fp2(), r.fp2()
    t = _dev_table(dev, alpha, g, log_len)
    torch.cuda.synchronize()
    want, absent = oracle.lookup_inverse_table(alpha, g, 1 << log_len)
    assert not absent.any()
    assert (t.cpu().numpy().view(np.uint64).reshape(-1, 2) == want).all()


def test_a_zero_denominator_is_an_absent_entry_and_refuses_only_where_carried(dev, oracle):
    import torch
    from intelligenceregulation_b200 import backend

    r = oracle.ZkRng(7, b"lookup-zero")
    g = r.fp2()
    hole = 201
    alpha = oracle.fp2_add((hole, 0), g)  # alpha - (201 + g) = 0
    t = _dev_table(dev, alpha, g, 8)
    torch.cuda.synchronize()
    want, absent = oracle.lookup_inverse_table(alpha, g, 256)
    assert absent.sum() == 1 and absent[hole]
    got = t.cpu().numpy().view(np.uint64).reshape(-1, 2)
    assert (got == want).all() and (got[hole] == 0).all()
    # a column that never carries the value: no refusal
    col = np.array([v for v in range(256) if v != hole] * 3, dtype=np.int64)
    re, im = _run(dev, col, t, 8, g, alpha)
    wre, wim = oracle.lookup_helpers(col, (want, absent), g, alpha)
    assert (re == wre).all() and (im == wim).all()
    # one carried occurrence: "zero LogUp denominator", in the first or the second column of a pair
    col2 = col.copy()
    col2[100] = hole
    assert oracle.lookup_helpers(col2, (want, absent), g, alpha) is None
    for a, b in ((col2, None), (col, col2), (col2, col)):
        with pytest.raises(backend.DeviceError) as e:
            _run(dev, a, t, 8, g, alpha, b=b, tb=t, lb=8, gb=g)
        assert e.value.code == -6
    # the same hole reached through the direct inversion of an out-of-table word: a 3-bit table, value 201 outside it
    t3 = _dev_table(dev, alpha, g, 3)
    with pytest.raises(backend.DeviceError) as e:
        _run(dev, np.array([1, 2, hole, 3]), t3, 3, g, alpha)
    assert e.value.code == -6


@pytest.mark.parametrize("n,log_len,paired", [(1, 8, False), (1000, 8, True), (1 << 20, 8, False), ((1 << 20) + 77, 8, True), (300000, 16, True), (5000, 16, False)])
def test_helper_planes(dev, oracle, n, log_len, paired):
    r = oracle.ZkRng(n + log_len, b"lookup-col")
    alpha, ga, gb = r.fp2(), r.fp2(), r.fp2()
    rng = np.random.default_rng(n)
    a = rng.integers(0, 1 << log_len, n).astype(np.int64)
    b = rng.integers(0, 256, n).astype(np.int64) if paired else None
    # tampered words: negative, beyond the table, beyond 2^32 (the direct inversion, protocol.rs:1172-1180)
    for k, v in enumerate((-1, 1 << log_len, -(1 << 40), (1 << 62) + 5, 70000)):
        if k < n:
            a[(k * 7919) % n] = v
    if paired and n > 3:
        b[3] = -77
    ta = _dev_table(dev, alpha, ga, log_len)
    oa = oracle.lookup_inverse_table(alpha, ga, 1 << log_len)
    tb = ob = None
    if paired:  # the second column in the byte table of another family (its own tag)
        tb = _dev_table(dev, alpha, gb, 8)
        ob = oracle.lookup_inverse_table(alpha, gb, 256)
    re, im = _run(dev, a, ta, log_len, ga, alpha, b=b, tb=tb, lb=8, gb=gb)
    wre, wim = oracle.lookup_helpers(a, oa, ga, alpha, b=b, tab_b=ob, g_b=gb)
    assert (re == wre).all() and (im == wim).all()


def test_arguments(dev):
    import torch
    from intelligenceregulation_b200 import backend

    t = torch.empty(512, dtype=torch.int64, device="cuda")
    with pytest.raises(backend.DeviceError) as e:
        dev.ctx.lookup_inverse_table((1, 2), (3, 4), 25, t.data_ptr())
    assert e.value.code == -7
    # an empty column is no work and no error
    dev.ctx.lookup_helpers_dev(t.data_ptr(), t.data_ptr(), 8, (1, 1), (5, 5), 0, 0, 0)
