"""Any slot polynomial on the device, given as data: the 23 slot graphs of the reference's recorded 125M shape
(structure from tests/golden/slot_ir_m125.json, coefficients and tables seeded) through `hl_b200_rounds_new_ir`,
compared with the CPU oracle's interpreter (private_block/slot_ir.rs:352-377) inside the oracle's masked sumcheck
driver: every unmasked round, every masked message, every challenge, the finals and the transcript end state.
Mirrors the reference's `ir_matches_closure` / evaluator contract tests (metal_slot.rs:483, sumcheck/rounds/tests.rs:65-142).
Field and hash work: bit-exact."""
import numpy as np
import pytest

import ir_util as U

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from intelligenceregulation_b200 import backend

    c = backend.Context(0)
    yield c
    c.close()


def _n_vars(slot):
    k = len(slot["table_fields"])
    return 13 if k <= 5 else 11 if k <= 25 else 10


# every slot at a size that runs the point form, the warp form and the single-CTA tail; three slots at sizes whose first
# rounds have more pairs than the machine has threads (the pair form)
CASES = [(i, None) for i in range(23)] + [(14, 16), (3, 17), (5, 16)]


@pytest.mark.parametrize("idx,n_long", CASES)
def test_slot_program_batched_masked_rounds(ctx, oracle, golden_dir, idx, n_long):
    from intelligenceregulation_b200 import backend

    o = oracle
    slot = U.load_slots(golden_dir)[idx]
    n, deg = n_long or _n_vars(slot), slot["declared_degree"]
    prog, _ = U.build_program(backend, slot, 9000 + idx)
    tables = U.random_tables(slot, n, 100 + idx)
    w, cf = prog.words(), prog.coef_array()
    o.ir_set(w, prog.n_nodes, prog.n_terms)
    coefs = cf if cf.size else None
    rng = o.ZkRng(300 + idx, b"slot-ir")
    mask = rng.fp2_vec((n + 1) * deg + 2)
    key = o.HashTag.for_profile("hashline-zk-mr1/b200-test/1").transcript
    tr = o.Transcript(b"b200-slot-ir", key)
    cc = tr.challenge_fp2()
    t_cpu = tr.clone()
    want = o.sc_prove(o.POLY_IR, tables, deg, t_cpu, coefs=coefs, mask=mask, mask_c=cc, mask_vars=n + 1)
    claim0 = o.fp2_add(tuple(map(int, want.rounds[0][0])), tuple(map(int, want.rounds[0][1])))
    ev = backend.B200Rounds(ctx, prog, tables, deg)
    sums, absorbed, ch, st, ctr, claim = ev.batched(n, tr.state, tr.counter, key, mask=mask, mask_vars=n + 1, mask_c=cc, recover_one=True, claim=claim0)
    assert (sums == want.rounds).all(), slot["name"]
    assert (absorbed == want.masked).all()
    assert (ch == want.challenges).all()
    assert st == t_cpu.state and ctr == t_cpu.counter
    assert (ev.finals() == want.finals).all()
    ev.free()


def test_slot_program_host_driven_rounds_equal_the_closed_form_family(ctx, oracle):
    """`impl SumcheckRounds` round by round: the LogUp query constraint written as a program returns the words of the
    built-in family, with and without the evaluation at 1."""
    from intelligenceregulation_b200 import backend

    SP = backend.SlotProgram
    o = oracle
    n = 14
    tables = o.ZkRng(11, b"ir-host").fp2_vec(3 << n).reshape(3, 1 << n, 2)
    alpha = (12345678901234567, 7654321)
    p = SP(3)
    a = p.affine(alpha, [(SP.NEG_ONE, 2)])
    s = p.sum([(SP.ONE, [1, SP.node(a)]), (SP.NEG_ONE, [])])
    p.term(SP.ONE, [0], [SP.node(s)])
    e_ir = backend.B200Rounds(ctx, p, tables, 3)
    e_bi = backend.B200Rounds(ctx, backend.POLY_LOGUP_Q, tables, 3, np.array([alpha], dtype=np.uint64))
    tr = o.Transcript(b"ir-host")
    for j in range(n):
        a_, b_ = e_ir.round(j, eval_one=(j % 2 == 0)), e_bi.round(j, eval_one=(j % 2 == 0))
        assert (a_ == b_).all(), j
        tr.absorb_fp2(b"sc-round", a_)
        r = tr.challenge_fp2()
        e_ir.fold(r)
        e_bi.fold(r)
    assert (e_ir.finals() == e_bi.finals()).all()
    e_ir.free()
    e_bi.free()


def test_malformed_program_is_refused_before_any_launch(ctx, oracle):
    from intelligenceregulation_b200 import backend

    SP = backend.SlotProgram
    tables = oracle.ZkRng(5, b"t").fp2_vec(2 * 8).reshape(2, 8, 2)
    p = SP(2)
    p.sum([(SP.ONE, [SP.node(0)])])  # a node that refers to itself
    p.term(SP.ONE, [0], [1])
    launches = ctx.stats()["kernel_launches"]
    with pytest.raises(backend.DeviceError):
        backend.B200Rounds(ctx, p, tables, 2)
    p = SP(2)
    p.term(SP.ONE, [0], [5])  # table id out of range
    with pytest.raises(backend.DeviceError):
        backend.B200Rounds(ctx, p, tables, 2)
    assert ctx.stats()["kernel_launches"] == launches
