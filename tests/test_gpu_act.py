"""The three-coordinate activation lookup on the device == the CPU restatement of accuracy_act.rs:13-117: multiplicities with
misses, query helpers, table values and table helper; the LogUp identity over hits; refusals.  Field and integer work: bit-exact."""
import numpy as np
import pytest
from act_util import instance

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from intelligenceregulation_b200 import backend

    c = backend.Context(0)
    yield c
    c.close()


@pytest.mark.parametrize("groups,f_pad,rows,tokens,hidden", [(1, 8, 3, 2, 5), (3, 64, 40, 33, 50), (4, 2048, 128, 128, 2048), (2, 16384, 128, 100, 14336)])
def test_histogram_helpers_table(ctx, oracle, groups, f_pad, rows, tokens, hidden):
    o = oracle
    tables, ids, gates, outputs = instance(groups + rows, groups, f_pad, rows, tokens, hidden)
    counts, misses = ctx.act_histogram(gates, outputs, f_pad, tokens, hidden, ids, tables)
    wc, wm = o.act_histogram(gates, outputs, f_pad, tokens, hidden, ids, tables)
    assert (counts == wc).all() and misses == wm and int(counts.sum()) == gates.size
    r = o.ZkRng(rows, b"act-gpu")
    alpha, beta, tag = r.fp2(), r.fp2(), r.fp2()
    h = ctx.act_helpers(gates, outputs, f_pad, tokens, hidden, ids, alpha, beta, tag)
    assert (h == o.act_helpers(gates, outputs, f_pad, tokens, hidden, ids, alpha, beta, tag)).all()
    length = 16384
    mult = np.zeros(length, dtype=np.uint64)
    mult[:groups * 4096] = counts
    comp, ht = ctx.act_table(tables, length, mult, alpha, beta, tag)
    wcomp, _ = o.act_table(tables, length, beta, tag)
    assert (comp == wcomp).all()
    den = np.stack([(int(alpha[0]) - wcomp[:, 0].astype(object)) % o._P0, (int(alpha[1]) - wcomp[:, 1].astype(object)) % o._P0], axis=1).astype(np.uint64)
    inv = o.batch_inverse2(den)
    want = np.array([o.fp2_mul_base((int(a), int(b)), int(m)) for (a, b), m in zip(inv, mult)], dtype=np.uint64)
    assert (ht == want).all()


def test_identity_over_an_honest_witness(ctx, oracle):
    # with no misses, sum of query helpers == sum of table helpers (protocol.rs:171-189)
    o = oracle
    tables, ids, gates, outputs = instance(3, 2, 64, 16, 16, 64, miss_every=10 ** 9)
    gates = np.clip(gates, -2048, 2047)
    idx = np.arange(gates.size)
    outputs = tables[ids[idx % 64], gates + 2048]
    counts, misses = ctx.act_histogram(gates, outputs, 64, 16, 64, ids, tables)
    assert misses == 0
    r = o.ZkRng(8, b"act-id")
    alpha, beta, tag = r.fp2(), r.fp2(), r.fp2()
    h = ctx.act_helpers(gates, outputs, 64, 16, 64, ids, alpha, beta, tag)
    mult = np.zeros(8192, dtype=np.uint64)
    mult[:] = counts
    _, ht = ctx.act_table(tables, 8192, mult, alpha, beta, tag)
    assert o.fp2_sub(o.fp2_sum(h), o.fp2_sum(ht)) == (0, 0)


def test_refusals(ctx, oracle):
    from intelligenceregulation_b200 import backend

    o = oracle
    tables, ids, gates, outputs = instance(4, 2, 64, 4, 4, 64)
    r = o.ZkRng(9, b"act-ref")
    beta, tag = r.fp2(), r.fp2()
    q = o.act_query_values(gates, outputs, 64, 4, 64, ids, beta, tag)
    with pytest.raises(backend.DeviceError) as e:
        ctx.act_helpers(gates, outputs, 64, 4, 64, ids, (int(q[100, 0]), int(q[100, 1])), beta, tag)
    assert e.value.code == -6
    with pytest.raises(backend.DeviceError) as e:  # rows must be whole
        ctx.act_helpers(gates[:-1], outputs[:-1], 64, 4, 64, ids, (1, 2), beta, tag)
    assert e.value.code == -1
    bad = tables.copy()
    bad[1, 2048] = 5
    with pytest.raises(backend.DeviceError) as e:  # "invalid generated table shape/zero row"
        ctx.act_table(bad, 8192, np.zeros(8192, dtype=np.uint64), (1, 2), beta, tag)
    assert e.value.code == -1
    with pytest.raises(backend.DeviceError) as e:  # the tables must fit in one row
        ctx.act_table(tables, 4096, np.zeros(4096, dtype=np.uint64), (1, 2), beta, tag)
    assert e.value.code == -1
