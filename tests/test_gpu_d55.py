"""D55 commit-fork-join with its work on the device (run_fork.rs:1617-1860): rank 0 commits the boundary planes and the roots
reach the other ranks in one broadcast; S1 after the join is the same whether one process proves every block or the blocks are
spread over ranks, one GPU each, with the join records exchanged by an NCCL all-gather.  The one-process case runs on any GPU box; the multi-rank case needs at least two GPUs and is skipped otherwise."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
P = 0xFFFFFFFF00000001
BLOCKS = 5


def header(d55):
    return d55.RunHeader(b"hashline-zk-mr1/d55-gpu-test/1", bytes(range(32)), BLOCKS, (128, 4096, 14336, 32, 8, 128), b"\x01" * 64, b"\x02" * 32,
                         b"params-line", b"\x03" * 16, b"\x04" * 32)


def block_inputs(k):
    rng = np.random.default_rng(9000 + k)
    lc, ir, rows, q, n = 10, 2, 40 + k, 16, 11
    nn = ir << lc
    pows, x = np.empty(nn, dtype=np.uint64), 1
    for i in range(nn):
        pows[i] = x
        x = x * 7 % P
    return dict(log_cols=lc, inv_rate=ir, data=rng.integers(0, P, rows << lc, dtype=np.uint64), pads=rng.integers(0, P, rows * q, dtype=np.uint64),
                salts=rng.integers(0, 256, (nn, 32), dtype=np.uint8), pows=pows, keys=(bytes(range(1, 33)), bytes(range(2, 34)), bytes(range(3, 35))),
                tables=rng.integers(0, P, (4, 1 << n, 2), dtype=np.uint64), mask=rng.integers(0, P, ((n + 1) * 3 + 2, 2), dtype=np.uint64))


def boundary_plane(dev, b):
    """the commitment of the plane between blocks b and b + 1: 38 rows of 2^10 words (32 data rows, two reserved row pairs, a
    proximity pair: boundary.rs:184-188), its salted root"""
    blk = block_inputs(100 + b)
    rows = 38
    st, _, levels = dev.try_commit_zk_tree(blk["log_cols"], blk["inv_rate"], blk["data"][: rows << blk["log_cols"]], blk["pads"][: rows * 16], blk["pows"], 11,
                                           blk["keys"][0], blk["salts"], blk["keys"][1], blk["keys"][2], want_leaves=False)
    st.free()
    return bytes(levels[-1])


def run(rank=0, world=1, all_gather=None, fail_block=None, broadcast=None):
    from intelligenceregulation_b200 import backend, d55

    dev = backend.B200Backend(device=rank if world > 1 else 0)
    roots = d55.commit_boundaries(lambda b: boundary_plane(dev, b), BLOCKS, rank, world, broadcast)
    digs = [bytes([50 + k]) * 32 for k in range(BLOCKS)]

    def prove(k, tr):
        if k == fail_block:
            raise RuntimeError("injected fork failure")
        return d55.device_fork(dev, backend, k, tr, block_inputs(k))

    try:
        return d55.run_forks(header(d55), roots, [38] * (BLOCKS - 1), [10] * (BLOCKS - 1), digs, prove, rank, world, all_gather)
    finally:
        dev.ctx.close()


def test_one_process_join_is_reproducible_and_sensitive_to_the_forks():
    from intelligenceregulation_b200 import d55

    a, b = run(), run()
    assert (a.state, a.counter) == (b.state, b.counter)
    with pytest.raises(d55.ForkFailed):
        run(fail_block=2)


WORKER = r'''
import os, sys
sys.path.insert(0, os.environ["HL_ROOT"]); sys.path.insert(0, os.path.join(os.environ["HL_ROOT"], "tests"))
import torch, torch.distributed as dist
import test_gpu_d55 as T
rank = int(os.environ["RANK"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
world = dist.get_world_size()
def gather(buf):
    mine = torch.tensor(list(buf), dtype=torch.uint8, device="cuda")
    out = torch.empty(world * mine.numel(), dtype=torch.uint8, device="cuda")
    dist.all_gather_into_tensor(out, mine)
    host = bytes(out.cpu().tolist())
    return [host[i * len(buf):(i + 1) * len(buf)] for i in range(world)]
def bcast(buf):
    n = 1 + 32 * (T.BLOCKS - 1)
    t = torch.tensor(list(buf), dtype=torch.uint8, device="cuda") if rank == 0 else torch.empty(n, dtype=torch.uint8, device="cuda")
    dist.broadcast(t, 0)
    return bytes(t.cpu().tolist())
s1 = T.run(rank, world, gather, broadcast=bcast)
open(os.path.join(os.environ["HL_OUT"], "rank%d.txt" % rank), "w").write("%s %d" % (s1.state.hex(), s1.counter))
dist.barrier()
dist.destroy_process_group()
'''


def test_two_ranks_on_two_gpus_join_to_the_one_process_state(tmp_path):
    import socket
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs (one rank per GPU)")
    want = run()
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, HL_ROOT=ROOT, HL_OUT=str(tmp_path), NCCL_NVLS_ENABLE="0")
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", str(port), str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    for rank in (0, 1):
        state, counter = (tmp_path / ("rank%d.txt" % rank)).read_text().split()
        assert state == want.state.hex() and int(counter) == want.counter
