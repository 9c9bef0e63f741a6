"""D55 commit-fork-join host logic on the CPU: the host transcript equals the oracle's, the join of a
two-rank gloo run equals the one-process join, and the reference's tamper controls change S1.

Modelled on the reference's run_fork_tests.rs (honest runs over several worker counts, fork-index swap,
unjoined claim); concurrency there is threads in one process, here ranks of a process group.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header(d55, key):
    return d55.RunHeader(b"hashline-zk-mr1/d55-test/1", key, 5, (128, 4096, 14336, 32, 8, 128), b"\x01" * 64, b"\x02" * 32,
                         b"params-line", b"\x03" * 16, b"\x04" * 32)


def _stub_fork(d55):
    """A stand-in for one block's proof: it drives the fork's transcript the way a proof does (absorbs,
    squeezes) and returns the join record.  Deterministic in (k, transcript)."""
    def prove(k, tr):
        tr.absorb(b"pb-slot", bytes([k]) * 40)
        for _ in range(3 + k):
            tr.challenge_fp2()
        ic = d55.claim_bytes([((k, 1), [(0, 19, (1, 0), [(5, 6)] * 19), (1 << 19, 14, (2, 3), [(7, 8)] * 14)])])
        oc = d55.claim_bytes([((k + 9, 2), [(4096, 19, (1, 0), [(9, 9)] * 19)])])
        return d55.JoinRecord(k, tr.state, tr.counter, ic, oc)
    return prove


def _inputs():
    roots = [bytes([10 + k]) * 32 for k in range(4)]
    return roots, [40] * 4, [14] * 4, [bytes([50 + k]) * 32 for k in range(5)]


def test_host_transcript_equals_the_oracle(oracle):
    from intelligenceregulation_b200 import d55

    for key in (None, oracle.HashTag.for_profile("hashline-zk-mr1/d55-test/1").transcript):
        a, b = d55.HostTranscript(b"dom", key), oracle.Transcript(b"dom", key)
        for i in range(6):
            data = bytes(range(256)) * i
            a.absorb(b"label-%d" % i, data)
            b.absorb(b"label-%d" % i, data)
            a.absorb_u64(b"rows", i * 977)
            b.absorb_u64(b"rows", i * 977)
            assert a.challenge_fp2() == b.challenge_fp2()
            assert a.state == b.state and a.counter == b.counter


def test_claim_list_length_formula():
    from intelligenceregulation_b200 import d55

    # one claim over the padded plane (19 coordinates) and the reserved pair's two parts (14 each): run_fork.rs:176-182
    c = [((1, 2), [(0, 19, (1, 0), [(0, 0)] * 19), (1, 14, (1, 0), [(0, 0)] * 14), (2, 14, (1, 0), [(0, 0)] * 14)])]
    assert len(d55.claim_bytes(c)) == d55.io_claim_list_len(19, 14)


def test_join_is_independent_of_the_world_size_and_catches_tampering(oracle):
    from intelligenceregulation_b200 import d55

    key = oracle.HashTag.for_profile("hashline-zk-mr1/d55-test/1").transcript
    h = _header(d55, key)
    roots, rows, logs, digs = _inputs()
    s1 = d55.run_forks(h, roots, rows, logs, digs, _stub_fork(d55))
    # two emulated ranks exchanging packed records
    cap = 4096
    bufs = []
    for rank in range(2):
        s0 = h.transcript()
        d55.absorb_commit(s0, h.blocks, roots, rows, logs)
        mine = [_stub_fork(d55)(k, d55.fork(s0, k, digs[k])) for k in d55.blocks_of(rank, 2, h.blocks)]
        bufs.append(b"".join(r.pack(cap) for r in mine).ljust(3 * d55.JoinRecord.size(cap), b"\xff"))
    s1b = d55.run_forks(h, roots, rows, logs, digs, _stub_fork(d55), rank=0, world=2, all_gather=lambda b: bufs, claim_cap=cap)
    assert s1.state == s1b.state and s1.counter == s1b.counter
    # the same absorbs through the oracle's transcript
    t = oracle.Transcript(h.profile, key)
    import struct
    t.absorb(b"run-shape", b"".join(struct.pack("<Q", v) for v in (h.blocks, *h.shape)))
    for lab, dat in ((b"expected-IO", h.expected_io), (b"public-statement", h.public_statement), (b"parameters", h.parameter_line),
                     (b"calibration", h.calibration), (b"schedule", h.schedule_digest)):
        t.absorb(lab, dat)
    for k, r in enumerate(roots):
        t.absorb_u64(b"pb-fork-commit-root", k); t.absorb(b"B", r); t.absorb_u64(b"rows", rows[k]); t.absorb_u64(b"log-cols", logs[k])
    t.absorb_u64(b"pb-fork-s0", h.blocks)
    recs = []
    for k in range(h.blocks):
        f = t.clone()
        f.absorb_u64(b"pb-run-fork", k); f.absorb(b"pb-run-fork-block", digs[k])
        f.absorb(b"pb-slot", bytes([k]) * 40)
        for _ in range(3 + k):
            f.challenge_fp2()
        recs.append((f.state, f.counter))
    s0 = h.transcript(); d55.absorb_commit(s0, h.blocks, roots, rows, logs)
    honest = [_stub_fork(d55)(k, d55.fork(s0, k, digs[k])) for k in range(h.blocks)]
    for k in range(h.blocks):
        assert (honest[k].state, honest[k].counter) == recs[k]
    # controls (run_fork_tests.rs ForkTamper): fork-index swap, stale state, missing fork
    swapped = list(honest); swapped[1], swapped[2] = (d55.JoinRecord(1, honest[2].state, honest[2].counter, honest[2].in_claims, honest[2].out_claims),
                                                      d55.JoinRecord(2, honest[1].state, honest[1].counter, honest[1].in_claims, honest[1].out_claims))
    assert d55.join(s0, swapped, h.blocks).state != s1.state
    stale = list(honest); stale[3] = d55.JoinRecord(3, honest[3].state, honest[3].counter + 1, honest[3].in_claims, honest[3].out_claims)
    assert d55.join(s0, stale, h.blocks).state != s1.state
    with pytest.raises(ValueError):
        d55.join(s0, honest[:-1], h.blocks)
    with pytest.raises(ValueError):
        d55.join(s0, honest[:-1] + [honest[0]], h.blocks)


WORKER = r'''
import os, sys
sys.path.insert(0, os.environ["HL_ROOT"]); sys.path.insert(0, os.path.join(os.environ["HL_ROOT"], "tests"))
import torch, torch.distributed as dist
from intelligenceregulation_b200 import d55
import test_d55_cpu as T
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
h = T._header(d55, bytes(range(32)))
roots, rows, logs, digs = T._inputs()
# rank 0 "commits" the boundary planes; the roots reach the other rank in one broadcast (d55.commit_boundaries)
def commit_plane(b):
    if os.environ.get("HL_FAIL_BOUNDARY") == str(b):
        raise RuntimeError("injected boundary failure")
    return roots[b]
def bcast(buf):
    n = 1 + 32 * (h.blocks - 1)
    t = torch.tensor(list(buf) if rank == 0 else [0] * n, dtype=torch.uint8)
    dist.broadcast(t, 0)
    return bytes(t.tolist())
try:
    roots = d55.commit_boundaries(commit_plane, h.blocks, rank, world, bcast)
except d55.ForkFailed as e:
    open(os.path.join(os.environ["HL_OUT"], "rank%d.txt" % rank), "w").write("FAILED " + str(e))
    dist.destroy_process_group()
    sys.exit(0)
def gather(buf):
    mine = torch.tensor(list(buf), dtype=torch.uint8)
    out = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(out, mine)
    return [bytes(o.tolist()) for o in out]
prove = T._stub_fork(d55)
if os.environ.get("HL_FAIL_BLOCK"):
    bad, good = int(os.environ["HL_FAIL_BLOCK"]), prove
    def prove(k, tr):
        if k == bad:
            raise RuntimeError("injected fork failure")
        return good(k, tr)
try:
    s1 = d55.run_forks(h, roots, rows, logs, digs, prove, rank, world, gather)
except d55.ForkFailed as e:
    open(os.path.join(os.environ["HL_OUT"], "rank%d.txt" % rank), "w").write("FAILED " + str(e))
    dist.destroy_process_group()
    sys.exit(0)
# one file per rank: the ranks share the launcher's pipe, where their output can interleave
open(os.path.join(os.environ["HL_OUT"], "rank%d.txt" % rank), "w").write("%s %d" % (s1.state.hex(), s1.counter))
dist.destroy_process_group()
'''


def _run_two_ranks(tmp_path, extra_env=None):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, HL_ROOT=ROOT, HL_OUT=str(tmp_path), OMP_NUM_THREADS="1", **(extra_env or {}))
    import socket

    for attempt in range(2):  # a free port can still be taken between the probe and the rendezvous: one retry
        with socket.socket() as sk:
            sk.bind(("127.0.0.1", 0))
            port = sk.getsockname()[1]
        out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                              "--master-port", str(port), str(script)], env=env, capture_output=True, text=True, timeout=300)
        if out.returncode == 0:
            break
    assert out.returncode == 0, out.stderr[-2000:]
    return [(tmp_path / ("rank%d.txt" % rank)).read_text() for rank in (0, 1)]


def test_two_rank_gloo_run_joins_to_the_one_process_state(tmp_path):
    from intelligenceregulation_b200 import d55

    h = _header(d55, bytes(range(32)))
    roots, rows, logs, digs = _inputs()
    want = d55.run_forks(h, roots, rows, logs, digs, _stub_fork(d55))
    for text in _run_two_ranks(tmp_path):
        state, counter = text.split()
        assert state == want.state.hex() and int(counter) == want.counter


def test_a_fork_that_fails_on_one_rank_ends_every_rank_with_the_same_error(tmp_path):
    """Block 1 belongs to rank 1 and its fork raises (a host-side failure: nothing on a device is involved).  Rank 1 still
    takes part in the exchange, so rank 0 does not wait in the gather for a peer that never comes; both ranks end promptly
    with the same `ForkFailed` text, which names the rank, the block and the cause."""
    import time

    t0 = time.time()
    texts = _run_two_ranks(tmp_path, {"HL_FAIL_BLOCK": "1"})
    assert time.time() - t0 < 120
    assert texts[0] == texts[1] and texts[0].startswith("FAILED D55: block 1 on rank 1: RuntimeError: injected fork failure")
    assert "block 3 on rank 1: not run" in texts[0]


def test_a_failed_fork_in_one_process_raises_fork_failed():
    from intelligenceregulation_b200 import d55

    h = _header(d55, None)
    roots, rows, logs, digs = _inputs()
    good = _stub_fork(d55)

    def prove(k, tr):
        if k == 2:
            raise ValueError("zero LogUp denominator")
        return good(k, tr)

    with pytest.raises(d55.ForkFailed) as ei:
        d55.run_forks(h, roots, rows, logs, digs, prove)
    assert ei.value.failures[0][:2] == (0, 2) and "zero LogUp denominator" in ei.value.failures[0][2]


def test_a_boundary_commitment_that_fails_on_rank_0_ends_every_rank(tmp_path):
    """Phase 1: rank 0 commits the boundary planes and broadcasts the roots.  A commitment that raises (a host-side failure) still
    takes part in the broadcast, so rank 1 does not wait for roots that never come; both ranks end with the same text."""
    texts = _run_two_ranks(tmp_path, {"HL_FAIL_BOUNDARY": "1"})
    assert texts[0] == texts[1] and texts[0].startswith("FAILED D55: block -1 on rank 0: RuntimeError: injected boundary failure")


def test_boundary_roots_in_one_process():
    from intelligenceregulation_b200 import d55

    roots = [bytes([b]) * 32 for b in range(4)]
    assert d55.commit_boundaries(lambda b: roots[b], 5) == roots
    assert d55.commit_boundaries(lambda b: roots[b], 1) == []
    with pytest.raises(d55.ForkFailed):
        d55.commit_boundaries(lambda b: (_ for _ in ()).throw(ValueError("no plane")), 3)
