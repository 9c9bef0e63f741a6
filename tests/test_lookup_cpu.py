"""The table form of the LogUp helper columns (oracle restatement of protocol.rs:1125-1230) against the element-wise form
it replaced: every helper word times its denominator is one, the words equal the whole-column batch inversion, a pair is
the sum of the two columns, and a zero denominator refuses only at a carried value — what the reference's own tests of
helper_inverses_u8 assert (protocol.rs tests of stage 28: table form == batch_inverse2_checked form)."""
import numpy as np


def _den(o, alpha, g, v):
    return o.fp2_sub(alpha, o.fp2_add((o.fp_from_i64(int(v)), 0), g))


def test_table_form_equals_elementwise(oracle):
    o = oracle
    r = o.ZkRng(3, b"lookup-cpu")
    alpha, g = r.fp2(), r.fp2()
    tab, absent = o.lookup_inverse_table(alpha, g, 256)
    assert not absent.any()
    for v in (0, 1, 17, 255):
        assert o.fp2_mul(tuple(int(x) for x in tab[v]), _den(o, alpha, g, v)) == (1, 0)
    col = np.array([0, 255, 3, 3, 99, -4, 256, 1 << 45], dtype=np.int64)
    re, im = o.lookup_helpers(col, (tab, absent), g, alpha)
    for i, v in enumerate(col):
        assert o.fp2_mul((int(re[i]), int(im[i])), _den(o, alpha, g, v)) == (1, 0)
    # the element-wise batch inversion of the same denominators (logup_helpers with beta = 0 is alpha - (idx + tag))
    small = np.array([5, 9, 200, 0], dtype=np.int32)
    h = o.logup_helpers(small, np.zeros(4, np.int32), alpha, (0, 0), g)
    re, im = o.lookup_helpers(small, (tab, absent), g, alpha)
    assert (h[:, 0] == re).all() and (h[:, 1] == im).all()
    # a pair is the sum
    b = np.array([1, 2, 3, 4], dtype=np.int64)
    pre, pim = o.lookup_helpers(small, (tab, absent), g, alpha, b=b, tab_b=(tab, absent), g_b=g)
    rb, ib = o.lookup_helpers(b, (tab, absent), g, alpha)
    for i in range(4):
        assert o.fp2_add((int(re[i]), int(im[i])), (int(rb[i]), int(ib[i]))) == (int(pre[i]), int(pim[i]))


def test_refusal_only_at_a_carried_value(oracle):
    o = oracle
    g = o.ZkRng(4, b"lookup-cpu").fp2()
    alpha = o.fp2_add((42, 0), g)
    tab, absent = o.lookup_inverse_table(alpha, g, 256)
    assert absent.sum() == 1 and absent[42] and (tab[42] == 0).all()
    assert o.lookup_helpers(np.array([1, 2, 41, 43]), (tab, absent), g, alpha) is not None
    assert o.lookup_helpers(np.array([1, 42]), (tab, absent), g, alpha) is None
    tab3 = o.lookup_inverse_table(alpha, g, 8)
    assert o.lookup_helpers(np.array([1, 42]), tab3, g, alpha) is None  # the direct inversion refuses as well
