"""Device sumcheck evaluator == CPU oracle / the reference's L6 agreement corpus, through the C ABI.

Follows the reference's evaluator contract tests (zkp-core/src/sumcheck/rounds/tests.rs:65-185: every
evaluator must reproduce the original prover's bytes, plain / masked / with recovery) and the device
Fiat-Shamir gate (slot_ir_accuracy.rs `m6_device_fiat_shamir_step_equals_the_transcript`).
Field and hash work: every comparison is bit-exact.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
P = 0xFFFFFFFF00000001


def fp2v(s):
    if s == "-":
        return np.zeros((0, 2), dtype=np.uint64)
    return np.array([int(x) for x in s.split(",")], dtype=np.uint64).reshape(-1, 2)


def f2(s):
    a, b = s.split(",")
    return (int(a), int(b))


def unhex(s):
    return b"" if s == "-" else bytes.fromhex(s)


@pytest.fixture(scope="module")
def ctx():
    from intelligenceregulation_b200 import backend

    c = backend.Context(0)
    yield c
    c.close()


def _blocks(golden_dir):
    cur = None
    for line in open(os.path.join(golden_dir, "l6_corpus.txt")):
        r = line.rstrip("\n").split(" ")
        if r[0] == "SCNEW":
            if cur:
                yield cur
            cur = []
        elif cur is not None and r[0].startswith("SC"):
            cur.append(r)
    if cur:
        yield cur


def prove_rounds(ev, tr, recover_claim=None, recover=False):
    """sumcheck/rounds.rs:33-48, host-driven: round -> absorb -> challenge -> fold."""
    rounds, chal, claim = [], [], recover_claim
    for j in range(ev.n_vars()):
        use = recover and claim is not None
        s = ev.round(j, eval_one=not use)
        if use:
            s[1] = _sub(claim, s[0])
        tr.absorb_fp2(b"sc-round", s)
        r = tr.challenge_fp2()
        if recover:
            claim = _interp(s, r)
        ev.fold(r)
        rounds.append(s)
        chal.append(r)
    return rounds, chal


_ORACLE = None


def _sub(a, b):
    return np.array(_ORACLE.fp2_sub(tuple(map(int, a)), tuple(map(int, b))), dtype=np.uint64)


def _interp(s, r):
    return _ORACLE.interpolate_eval(s, r)


def test_l6_corpus_sumchecks_on_the_device(ctx, oracle, golden_dir):
    """Every honest sumcheck of the L6 corpus re-proved with the tables on the device: host-driven rounds
    for the plain ones (with and without s(1) recovery), one device batch for the masked ones."""
    global _ORACLE
    _ORACLE = o = oracle
    from intelligenceregulation_b200 import backend

    done = 0
    for blk in _blocks(golden_dir):
        if not any(r[0] in ("SCFIN", "SCMFIN", "SCEXT") for r in blk):
            continue
        tables = np.stack([fp2v(r[1]) for r in blk if r[0] == "SCTAB"])
        mask = next((r for r in blk if r[0] == "SCMASK"), None)
        fin = next(r for r in blk if r[0] in ("SCFIN", "SCMFIN", "SCEXT"))
        poly = {"prod": backend.POLY_PROD, "zc": backend.POLY_ZC}[fin[1]]
        h = next(r for r in blk if r[0] == "SC")
        domain, key, deg = unhex(h[2]), (None if h[3] == "-" else bytes.fromhex(h[3])), int(h[4])
        scr, end = [], None
        for r in blk:
            if r[0] == "SCR" and end is None:
                scr.append(fp2v(r[1]))
            elif r[0] == "SCEND" and end is None:
                end = r
        n = tables.shape[1].bit_length() - 1
        if n == 0:
            continue
        tr = o.Transcript(domain, key)
        if mask is None:
            for recover in (False, True):
                t = tr.clone()
                ev = backend.B200Rounds(ctx, poly, tables, deg)
                rounds, chal = prove_rounds(ev, t, None, recover)
                for j in range(n):
                    assert (rounds[j] == scr[j]).all(), (h[1], j, recover)
                assert (ev.finals() == fp2v(fin[2])).all()
                assert t.state.hex() == end[-1]
                ev.free()
            # and the same rounds as ONE device batch (no mask), from the same transcript position
            ev = backend.B200Rounds(ctx, poly, tables, deg)
            sums, absorbed, ch, st, ctr, _ = ev.batched(n, tr.state, tr.counter, key, recover_one=True)
            assert all((sums[j] == scr[j]).all() and (absorbed[j] == scr[j]).all() for j in range(n))
            assert st.hex() == end[-1] and ctr == tr.counter + n
            assert (ev.finals() == fp2v(fin[2])).all()
            ev.free()
        else:
            cc = tr.challenge_fp2()
            mv, md, mco = int(mask[1]), int(mask[2]), fp2v(mask[3])
            unm = [fp2v(r[2]) for r in blk if r[0] == "SCUNM"]
            for recover in (False, True):
                ev = backend.B200Rounds(ctx, poly, tables, deg)
                sums, absorbed, ch, st, ctr, _ = ev.batched(n, tr.state, tr.counter, key, mask=mco, mask_vars=mv, mask_c=cc, recover_one=recover)
                for j in range(n):
                    assert (sums[j] == unm[j]).all(), (h[1], j)
                    assert (absorbed[j] == scr[j]).all(), (h[1], j)
                # the host replay the reference performs on every device round (metal.rs:4156-4171)
                t = tr.clone()
                for j in range(n):
                    t.absorb_fp2(b"sc-round", absorbed[j])
                    assert t.challenge_fp2() == tuple(map(int, ch[j]))
                assert t.state == st and t.counter == ctr
                assert (ev.finals() == fp2v(fin[2])).all()
                ev.free()
        done += 1
    assert done >= 14


@pytest.mark.parametrize("poly_name,k,deg,n", [("prod", 2, 2, 12), ("zc", 4, 3, 16), ("prod", 3, 3, 14), ("logup_q", 3, 3, 15), ("logup_t", 4, 3, 13),
                                               ("prod", 6, 6, 11), ("prod", 1, 1, 17), ("zc", 4, 3, 20), ("logup_q", 3, 3, 19)])
def test_random_cubes_masked_batches_match_the_oracle(ctx, oracle, poly_name, k, deg, n):
    """Larger cubes (many CTAs per round, partial-sum trees) against the oracle's prover, masked, keyed, with the running claim
    from the first round on, and (second run) without claim recovery in two batches, where the point 1 is evaluated in every round
    and the second batch starts in the middle of the long rounds."""
    o = oracle
    from intelligenceregulation_b200 import backend


    poly = {"prod": 0, "zc": 1, "logup_q": 2, "logup_t": 3}[poly_name]
    rng = o.ZkRng(1000 + n, b"b200-sumcheck-test")
    tables = rng.fp2_vec(k * (1 << n)).reshape(k, 1 << n, 2)
    coefs = rng.fp2_vec(1) if poly >= 2 else None
    mask = rng.fp2_vec((n + 1) * deg + 2)
    key = o.HashTag.for_profile("hashline-zk-mr1/b200-test/1").transcript
    tr = o.Transcript(b"b200-sumcheck", key)
    cc = tr.challenge_fp2()
    t_cpu = tr.clone()
    want = o.sc_prove(poly, tables, deg, t_cpu, coefs=coefs, mask=mask, mask_c=cc, mask_vars=n + 1)
    ev = backend.B200Rounds(ctx, poly, tables, deg, coefs)
    # the exact unmasked sum of round 0, so that recovery starts at once (rounds.rs:81-86)
    claim0 = o.fp2_add(tuple(map(int, want.rounds[0][0])), tuple(map(int, want.rounds[0][1])))
    sums, absorbed, ch, st, ctr, claim = ev.batched(n, tr.state, tr.counter, key, mask=mask, mask_vars=n + 1, mask_c=cc, recover_one=True, claim=claim0)
    assert (sums == want.rounds).all()
    assert (absorbed == want.masked).all()
    assert (ch == want.challenges).all()
    assert st == t_cpu.state and ctr == t_cpu.counter
    assert (ev.finals() == want.finals).all()
    assert claim == o.interpolate_eval(want.rounds[-1], tuple(map(int, want.challenges[-1])))
    ev.free()
    if n <= 17:  # no recovery, no mask, in two batches: the second one starts in the middle of the long rounds
        t2 = tr.clone()
        want = o.sc_prove(poly, tables, deg, t2, coefs=coefs)
        ev = backend.B200Rounds(ctx, poly, tables, deg, coefs)
        first = max(1, n - 11)
        a_ = ev.batched(first, tr.state, tr.counter, key)
        b_ = ev.batched(n - first, a_[3], a_[4], key)
        assert (np.concatenate([a_[0], b_[0]]) == want.rounds).all() and b_[3] == t2.state
        assert (ev.finals() == want.finals).all()
        ev.free()


def test_round_order_is_enforced(ctx, oracle):
    """rounds.rs:95-96: a round needs the preceding fold; finals need all folds."""
    from intelligenceregulation_b200 import backend

    tables = oracle.ZkRng(5, b"t").fp2_vec(2 * 8).reshape(2, 8, 2)
    ev = backend.B200Rounds(ctx, 0, tables, 2)
    with pytest.raises(backend.DeviceError):
        ev.round(1)
    with pytest.raises(backend.DeviceError):
        ev.finals()
    ev.round(0)
    ev.free()
    with pytest.raises(backend.DeviceError):
        backend.B200Rounds(ctx, 1, tables, 3)  # zc needs four tables
