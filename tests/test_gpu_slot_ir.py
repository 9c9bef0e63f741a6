"""Any slot polynomial on the device, given as data: the 23 slot graphs of the reference's recorded 125M shape
(structure from tests/golden/slot_ir_m125.json, coefficients and tables seeded) through `hl_b200_rounds_new_ir`,
compared with the CPU oracle's interpreter (private_block/slot_ir.rs:352-377) inside the oracle's masked sumcheck
driver: every unmasked round, every masked message, every challenge, the finals and the transcript end state.
Mirrors the reference's `ir_matches_closure` / evaluator contract tests (metal_slot.rs:483, sumcheck/rounds/tests.rs:65-142).
Field and hash work: bit-exact."""
import numpy as np
import pytest

import ir_util as U

P_ = 0xFFFFFFFF00000001

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
# rounds have more pairs than the machine has threads (the pair form); the D zero-check at its 8B size of 2^19 points and the
# softmax zero-check at 2^20, the sizes the benchmark times
CASES = [(i, None) for i in range(23)] + [(14, 16), (3, 17), (5, 16), (14, 19), (17, 20)]


@pytest.mark.parametrize("generated", [True, False])
@pytest.mark.parametrize("idx,n_long", CASES)
def test_slot_program_batched_masked_rounds(ctx, oracle, golden_dir, idx, n_long, generated):
    """`generated`: the per-graph compiled kernel the library holds for each of these graphs, or the interpreter that serves any
    graph (both must return the oracle's words; the largest sizes run once, through the generated kernels)"""
    from intelligenceregulation_b200 import backend

    if not generated and (n_long or 0) >= 19:
        pytest.skip("the largest sizes run through the generated kernels only")
    ctx.set_slot_kernels(generated)
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
    ctx.set_slot_kernels(False)


def test_every_known_graph_has_its_generated_kernel(ctx, oracle, golden_dir):
    """The dispatcher recognises all 23 recorded graphs and all 23 graphs of the real W16R2 core by their signature (the word
    stream with coefficient classes in place of values): with the generated kernels on, a short sumcheck over each of them
    launches exactly the round kernel, the step and the fold per multi-CTA round that the generated path launches, and with
    random tables in place of base-valued ones (so that the first-round typing does not apply) the words still equal the
    interpreter's."""
    from intelligenceregulation_b200 import backend
    import l11_util

    o = oracle
    progs = [(U.build_program(backend, s, 7000 + i)[0], s["declared_degree"], len(s["table_fields"])) for i, s in enumerate(U.load_slots(golden_dir))]
    progs += [(l11_util.build_program(backend, s)[0], s["degree"], s["n_tabs"]) for s in l11_util.load(golden_dir)["slots"]]
    n = 14  # above every program's one-CTA tail, so that at least two rounds run as grid launches
    for j, (prog, deg, k) in enumerate(progs):
        tables = o.ZkRng(600 + j, b"gen-any").fp2_vec(k << n).reshape(k, 1 << n, 2)  # every table extension-valued
        outs = []
        for gen in (True, False):
            ctx.set_slot_kernels(gen)
            before = ctx.stats()["generated_rounds"]
            ev = backend.B200Rounds(ctx, prog, tables, deg)
            outs.append(ev.batched(n, bytes(32), 5, None)[0])
            ev.free()
            assert (ctx.stats()["generated_rounds"] > before) == gen, (j, gen)
        assert (outs[0] == outs[1]).all(), j
    ctx.set_slot_kernels(False)


def test_plan_beyond_the_all_points_form_runs_the_stepping_pair_form(ctx, oracle):
    """A polynomial with more non-affine nodes than the all-points pair-per-thread kernel keeps (40) at 2^15 points: its long
    rounds run the stepping form (`k_sc_round_irp`), which none of the recorded graphs reaches.  A chain of 44 sum nodes over
    four tables, each node the product of the previous node's affine image and a table plus a second unit, so that every node
    matters; compared with the oracle's masked prover word for word."""
    from intelligenceregulation_b200 import backend

    SP, o = backend.SlotProgram, oracle
    n, deg = 15, 3
    rng = o.ZkRng(77, b"irp")
    cf = [tuple(map(int, c)) for c in rng.fp2_vec(100)]
    p = SP(4)
    a0 = p.affine(cf[0], [(cf[1], 1), (SP.NEG_ONE, 2)])
    prev = p.sum([(SP.ONE, [1, 2]), (cf[2], [3])])
    for i in range(43):  # degree stays 2: each node is linear in the tables through one product of two affine-type factors
        prev = p.sum([(cf[3 + i], [1 + (i % 3), SP.node(a0)]), (cf[50 + i], [1 + ((i + 1) % 3)]), (SP.ONE, [])] if i % 2 else
                     [(cf[3 + i], [2, 3]), (SP.NEG_ONE, [SP.node(a0)])])
    mix = p.sum([(cf[90], [SP.node(prev)]), (cf[91], [SP.node(prev - 1)]), (cf[92], [SP.node(prev - 2)]), (cf[93], [SP.node(prev - 3)])])
    p.term(SP.ONE, [0], [SP.node(mix)])
    tables = rng.fp2_vec(4 << n).reshape(4, 1 << n, 2)
    tables[2, :, 1] = 0
    w, c = p.words(), p.coef_array()
    o.ir_set(w, p.n_nodes, p.n_terms)
    mask = rng.fp2_vec((n + 1) * deg + 2)
    tr = o.Transcript(b"irp")
    cc = tr.challenge_fp2()
    t_cpu = tr.clone()
    want = o.sc_prove(o.POLY_IR, tables, deg, t_cpu, coefs=c, mask=mask, mask_c=cc, mask_vars=n + 1)
    claim0 = o.fp2_add(tuple(map(int, want.rounds[0][0])), tuple(map(int, want.rounds[0][1])))
    ev = backend.B200Rounds(ctx, p, tables, deg)
    sums, absorbed, ch, st, ctr, _ = ev.batched(n, tr.state, tr.counter, None, mask=mask, mask_vars=n + 1, mask_c=cc, recover_one=True, claim=claim0)
    assert (sums == want.rounds).all() and (absorbed == want.masked).all() and st == t_cpu.state
    assert (ev.finals() == want.finals).all()
    ev.free()
    # the same without claim recovery: the point 1 is evaluated too
    ev = backend.B200Rounds(ctx, p, tables, deg)
    t2 = tr.clone()
    want = o.sc_prove(o.POLY_IR, tables, deg, t2, coefs=c)
    sums = ev.batched(n, tr.state, tr.counter, None)[0]
    assert (sums == want.rounds).all()
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


# ----------------------------------------------------------------------------- the reference's own numbers (L11 corpus)
def _l11(golden_dir):
    import l11_util

    return l11_util.load(golden_dir)["slots"]


@pytest.mark.parametrize("idx", range(23))
def test_l11_recorded_graphs_reach_the_reference_value_on_the_device(ctx, oracle, golden_dir, idx):
    """Each slot graph of the reference's real W16R2 block core, with its RECORDED coefficient values, evaluated by the device at
    the recorded terminal values `VALS`: the sums must be the reference's own `poly(vals)` (lean_l11_export_tests.rs:243,
    `RES`).  Three shapes per slot: one pair whose low entry is `VALS` (s(0) is the recorded value itself; s(1) is checked by
    the independent Python walk), constant tables at a size that runs the warp form and the one-CTA tail (every s(d) is
    2^(n-1) times the recorded value, and the finals after the folds are `VALS` again), and the same at 2^16 points, which
    runs the pair-per-thread form."""
    from intelligenceregulation_b200 import backend
    import l11_util

    o = oracle
    s = _l11(golden_dir)[idx]
    prog, desc = l11_util.build_program(backend, s)
    deg, k = s["degree"], s["n_tabs"]
    vals = np.array(s["vals"], dtype=np.uint64)
    rng = np.random.default_rng(4100 + idx)
    other = rng.integers(0, P_, size=(k, 2), dtype=np.uint64)
    tables = np.stack([vals, other], axis=1)  # (k, 2, 2): entry 0 = VALS, entry 1 = its pair
    ev = backend.B200Rounds(ctx, prog, tables, deg)
    got = ev.round(0)
    assert tuple(map(int, got[0])) == s["pv"], ("s(0)", idx)
    assert tuple(map(int, got[1])) == U.py_eval(desc, [tuple(map(int, x)) for x in other]), ("s(1)", idx)
    ev.free()
    for n in (11, 16):
        tables = np.repeat(vals[:, None, :], 1 << n, axis=1)
        ev = backend.B200Rounds(ctx, prog, tables, deg)
        tr = o.Transcript(b"l11-const")
        for j in range(n):
            got = ev.round(j)
            want_j = o.fp2_mul_base(s["pv"], 1 << (n - 1 - j))
            assert all(tuple(map(int, g)) == want_j for g in got), (idx, n, j)
            tr.absorb_fp2(b"sc-round", got)
            ev.fold(tr.challenge_fp2())
        assert (ev.finals() == vals).all()
        ev.free()


def test_l11_recorded_rounds_replay_on_the_device_transcript(ctx, oracle, golden_dir):
    """The device Fiat-Shamir step against the reference's recorded transcript: for every slot, constant tables whose round
    messages are known in closed form are proved by the device from the recorded state `TRB` (after `pb-slot`, the slot
    challenge and `pb-scalar`, which the caller absorbs), and the oracle's verifier, replaying from the same recorded state,
    accepts them and ends in the device's state."""
    from intelligenceregulation_b200 import backend
    import l11_util

    o = oracle
    corpus = l11_util.load(golden_dir)
    key = corpus["head"]["key"]
    for s in corpus["slots"][:8]:
        prog, _ = l11_util.build_program(backend, s)
        deg, n = s["degree"], 9
        vals = np.array(s["vals"], dtype=np.uint64)
        tr = o.Transcript.from_state(*s["trb"], key=key)
        tr.absorb_u64(b"pb-slot", s["slot"])
        assert tr.challenge_fp2() == s["c"]
        tr.absorb_fp2(b"pb-scalar", np.array([s["scalar"]], dtype=np.uint64))
        tables = np.repeat(vals[:, None, :], 1 << n, axis=1)
        ev = backend.B200Rounds(ctx, prog, tables, deg)
        claim = o.fp2_mul_base(s["pv"], 1 << n)
        sums, absorbed, ch, st, ctr, _ = ev.batched(n, tr.state, tr.counter, key, recover_one=True, claim=claim)
        got, err = o.sc_verify(claim, deg, n, [x for x in absorbed], tr)
        assert err is None, err
        assert (tr.state, tr.counter) == (st, ctr)
        assert [tuple(map(int, r)) for r in got[1]] == [tuple(map(int, r)) for r in ch]
        assert (ev.finals() == vals).all() and got[0] == s["pv"]
        ev.free()
