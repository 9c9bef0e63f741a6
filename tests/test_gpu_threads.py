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


def test_threads_that_decline_do_not_disturb_the_ones_that_work():
    """Declines are routine in a fork run (a shape the device refuses, an argument check): two threads provoke them without
    pause, two others read the error text, and two work.  The error text and the decline counter have their own lock, so the
    workers' results still equal the serial ones and every error text read is a whole message."""
    from intelligenceregulation_b200 import backend

    dev = backend.B200Backend(device=0)
    seeds = [5, 6]
    serial = [_work(dev, backend, s) for s in seeds]
    stop = threading.Event()
    errs, texts = [], set()

    def decliner(k):
        tables = np.zeros((2, 8, 2), dtype=np.uint64)
        while not stop.is_set():
            try:
                if k == 0:
                    assert dev.try_commit(30, 2, np.zeros(4, dtype=np.uint64), 31) is None  # rows of 2^30 words: unsupported
                else:
                    backend.B200Rounds(dev.ctx, backend.POLY_ZC, tables, 7)  # the zero-check family has 4 tables, degree 3
                    errs.append("an unsupported family was accepted")
            except backend.DeviceError:
                pass
            except Exception as e:
                errs.append(e)

    def reader():
        while not stop.is_set():
            texts.add(dev.ctx.last_error())

    got = [None] * len(seeds)

    def worker(i):
        try:
            for _ in range(3):
                got[i] = _work(dev, backend, seeds[i])
                assert got[i] == serial[i]
        except Exception as e:
            errs.append(e)

    side = [threading.Thread(target=decliner, args=(k,)) for k in (0, 1)] + [threading.Thread(target=reader) for _ in range(2)]
    work = [threading.Thread(target=worker, args=(i,)) for i in range(len(seeds))]
    for t in side + work:
        t.start()
    for t in work:
        t.join()
    stop.set()
    for t in side:
        t.join()
    assert not errs, errs
    assert got == serial
    assert dev.ctx.stats()["declines"] > 0
    assert all(t.isprintable() and len(t) < 200 for t in texts), texts
    dev.ctx.close()


def test_one_context_per_thread_on_one_gpu_equals_the_serial_results():
    """The arrangement the header recommends for concurrent forks: every worker thread owns a context (its own stream,
    twiddle tables and staging) on the same GPU, so that their calls overlap instead of queueing behind one lock."""
    from intelligenceregulation_b200 import backend

    seeds = [1, 2, 3, 4]
    ref = backend.B200Backend(device=0)
    serial = [_work(ref, backend, s) for s in seeds]
    ref.ctx.close()
    got, errs = [None] * len(seeds), []

    def run(i):
        try:
            dev = backend.B200Backend(device=0)
            for _ in range(3):
                got[i] = _work(dev, backend, seeds[i])
                assert got[i] == serial[i]
            assert not dev.ctx.declines
            dev.ctx.close()
        except Exception as e:
            errs.append(e)

    th = [threading.Thread(target=run, args=(i,)) for i in range(len(seeds))]
    for t in th:
        t.start()
    for t in th:
        t.join()
    assert not errs, errs
    assert got == serial
