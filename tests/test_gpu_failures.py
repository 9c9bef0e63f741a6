"""Decline / refusal behaviour of the device backend, with every failure made on the host.

The reference's seam treats an accelerator error as a decline (hashline/src/gpu/mod.rs:80-94) that is fatal
under HL_GPU_REQUIRED=1 (:76-78), and its CUDA tests inject allocation failures
(tests/zk60_gpu_commit.rs, mod.rs:121).  Nothing here faults, traps or hangs the GPU.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
P = 0xFFFFFFFF00000001


@pytest.fixture()
def dev():
    from intelligenceregulation_b200 import backend

    b = backend.B200Backend()
    yield b
    b.ctx.close()


def _data(n):
    return (np.arange(1, n + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)) % np.uint64(P)


def test_allocation_failure_is_a_decline_and_the_context_survives(dev, oracle, monkeypatch):
    from intelligenceregulation_b200 import backend

    log_cols, ir, rows, q = 10, 4, 64, 16
    n, nn = 1 << log_cols, (1 << log_cols) * ir
    data, pads, pows = _data(rows * n), _data(rows * q), oracle.coset_powers(7, nn)
    dev.ctx.set_alloc_cap(1 << 20)  # the encoding alone is 2 MiB
    assert dev.try_commit_zk(log_cols, ir, data, pads, pows, 12) is None
    assert dev.ctx.declines and "cap" in dev.ctx.declines[-1][1]
    monkeypatch.setenv("HL_GPU_REQUIRED", "1")
    with pytest.raises(backend.DeviceError) as e:
        dev.try_commit_zk(log_cols, ir, data, pads, pows, 12)
    assert e.value.code == -2
    monkeypatch.delenv("HL_GPU_REQUIRED")
    dev.ctx.set_alloc_cap(0)
    store, leaves = dev.try_commit_zk(log_cols, ir, data, pads, pows, 12)
    enc = oracle.encode_rows_zk(data, rows, n, pads, q, pows, 12)
    assert (leaves == oracle.hash_columns(enc, rows, nn)).all()
    assert dev.ctx.stats()["declines"] >= 2
    store.free()


def test_shapes_outside_the_kernels_range_decline(dev, oracle):
    assert dev.try_commit(17, 2, np.zeros(1 << 17, dtype=np.uint64), 18) is None          # rows of 2^17 words
    assert dev.try_commit(10, 3, np.zeros(1 << 10, dtype=np.uint64), 12) is None          # rate not a power of two
    assert dev.try_commit(10, 4, np.zeros(1 << 10, dtype=np.uint64), 11) is None          # beyond the caller's NTT tables
    pows = oracle.coset_powers(7, 1 << 11)
    assert dev.try_commit_zk(10, 2, np.zeros(1 << 10, dtype=np.uint64), np.zeros(1025, dtype=np.uint64), pows, 11) is None  # n + q > nn
    assert len(dev.ctx.declines) == 4


def test_single_row_and_single_chunk_edges(dev, oracle):
    for log_cols, ir, rows in ((1, 2, 1), (2, 4, 3), (8, 2, 1), (14, 2, 2)):
        n, nn = 1 << log_cols, (1 << log_cols) * ir
        data = _data(rows * n)
        store, leaves = dev.try_commit(log_cols, ir, data, 16)
        enc = oracle.encode_rows_plain(data, rows, n, nn, 16)
        assert (leaves == oracle.hash_columns(enc, rows, nn)).all()
        assert (store.columns(np.arange(nn, dtype=np.uint64)).T.reshape(-1) == enc).all()
        assert store.columns(np.zeros(0, dtype=np.uint64)).shape == (0, rows)
        store.free()


def test_misaligned_caller_device_pointers_are_a_bad_argument_not_a_fault(dev, oracle):
    """Device pointers that the kernels would move as 16-byte vectors are checked on the host: the call answers
    HL_B200_ERR_ARG and launches nothing."""
    import ctypes as C
    import torch
    from intelligenceregulation_b200 import backend

    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    base = buf.data_ptr()
    assert base % 16 == 0
    log_cols, ir, rows = 8, 2, 4
    store, _ = dev.try_commit(log_cols, ir, _data(rows << log_cols), 10)
    launches = dev.ctx.stats()["kernel_launches"]
    with pytest.raises(backend.DeviceError) as e:
        dev.ctx.lookup_inverse_table((5, 6), (7, 8), 8, base + 8)
    assert e.value.code == -1
    with pytest.raises(backend.DeviceError) as e:
        store.merkle_dev(base + 4, None, None, base + 4096)
    assert e.value.code == -1
    with pytest.raises(backend.DeviceError) as e:
        store.merkle_dev(base, None, None, base + 4096 + 8)
    assert e.value.code == -1
    assert dev.ctx.stats()["kernel_launches"] == launches
    store.free()
    del buf
