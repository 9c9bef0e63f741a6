"""The CPU restatement of accuracy_act.rs:13-117 against itself in the two forms the reference keeps (query_values and
denominators give alpha - q word for word; the histogram counts every query; the table's padding entries are 2048 + tag)."""
import numpy as np
from act_util import instance


def test_forms_agree(oracle):
    o = oracle
    groups, f_pad, rows, tokens, hidden = 3, 64, 40, 33, 50
    tables, ids, gates, outputs = instance(1, groups, f_pad, rows, tokens, hidden)
    counts, misses = o.act_histogram(gates, outputs, f_pad, tokens, hidden, ids, tables)
    assert int(counts.sum()) == gates.size and misses > 0 and counts[0] >= misses
    r = o.ZkRng(2, b"act")
    alpha, beta, tag = r.fp2(), r.fp2(), r.fp2()
    q = o.act_query_values(gates, outputs, f_pad, tokens, hidden, ids, beta, tag)
    h = o.act_helpers(gates, outputs, f_pad, tokens, hidden, ids, alpha, beta, tag)
    for i in (0, 5, 7, 63, 64 * 33 + 1, gates.size - 1):
        d = o.fp2_sub(alpha, (int(q[i, 0]), int(q[i, 1])))
        assert o.fp2_mul(d, (int(h[i, 0]), int(h[i, 1]))) == (1, 0)
        # the expression itself, from the reference's text
        live = i // f_pad < tokens and i % f_pad < hidden
        want = o.fp2_add(o.fp2_add(o.fp2_add((o.fp_add(o.fp_from_i64(int(gates[i])), 2048), 0), o.fp2_mul_base(beta, o.fp_from_i64(int(outputs[i])))),
                                   o.fp2_mul_base(o.fp2_mul(beta, beta), int(ids[i % f_pad]) if live else 0)), tag)
        assert want == (int(q[i, 0]), int(q[i, 1]))
    comp, sup = o.act_table(tables, 16384, beta, tag)
    assert tuple(int(x) for x in comp[groups * 4096]) == o.fp2_add((2048, 0), tag) and not sup[groups * 4096:].any() and (sup[:groups * 4096, 0] == 1).all()
    # a hit's query value is its table entry: the LogUp identity's premise
    i = 1
    g = int(ids[i % f_pad])
    assert (q[i] == comp[g * 4096 + int(gates[i]) + 2048]).all()
    # a zero denominator refuses
    assert o.act_helpers(gates, outputs, f_pad, tokens, hidden, ids, (int(q[9, 0]), int(q[9, 1])), beta, tag) is None
