"""Concurrent callers: the reference's fork workers call into one process-wide device context from several threads at
once (run_fork.rs:1677-1779; the context and its buffer pool sit behind a mutex, gpu/metal.rs:386).  Four threads share
ONE context and each commits, opens and runs a sumcheck on its own inputs; every result must equal the single-thread
result of the same inputs (the reference's thread-count-independence gates: transcript.rs:401-406, slot_ir_tests.rs:181)."""
import threading

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
P = 0xFFFFFFFF00000001


def _work(dev, backend, seed):
    rng = np.random.default_rng(seed)
    log_cols, ir, rows, q = 9 + seed % 3, 4, 40 + 7 * seed, 24
    n, nn = 1 << log_cols, (1 << log_cols) * ir
    data = rng.integers(0, P, size=rows * n, dtype=np.uint64)
    pads = rng.integers(0, P, size=rows * q, dtype=np.uint64)
    pows = rng.integers(0, P, size=nn, dtype=np.uint64)
    key = bytes(rng.integers(0, 256, size=32, dtype=np.uint8))
    store, leaves = dev.try_commit_zk_keyed(log_cols, ir, data, pads, pows, 14, key)
    rhos = rng.integers(0, P, size=(5, rows, 2), dtype=np.uint64)
    fold = store.fold_rows_with_pads(rhos)
    cols = store.columns(rng.integers(0, nn, size=17, dtype=np.uint64))
    store.free()
    tables = rng.integers(0, P, size=(4, 1 << 13, 2), dtype=np.uint64)
    ev = backend.B200Rounds(dev.ctx, backend.POLY_ZC, tables, 3)
    out = ev.batched(13, bytes(32), seed, None, recover_one=False)
    fin = ev.finals()
    ev.free()
    return leaves.tobytes(), fold.tobytes(), cols.tobytes(), out[0].tobytes(), out[2].tobytes(), out[3], fin.tobytes()


def test_four_threads_on_one_context_equal_the_serial_results():
    from intelligenceregulation_b200 import backend

    dev = backend.B200Backend(device=0)
    seeds = [1, 2, 3, 4]
    serial = [_work(dev, backend, s) for s in seeds]
    for _ in range(3):
        got = [None] * len(seeds)
        errs = []

        def run(i):
            try:
                got[i] = _work(dev, backend, seeds[i])
            except Exception as e:  # a failure in a worker must fail the test, not vanish with the thread
                errs.append(e)

        th = [threading.Thread(target=run, args=(i,)) for i in range(len(seeds))]
        for t in th:
            t.start()
        for t in th:
            t.join()
        assert not errs, errs
        assert got == serial
    assert not dev.ctx.declines
    dev.ctx.close()
