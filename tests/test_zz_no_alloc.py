"""The allocation-free column hash (hl_b200_hash_columns_static) against the regular commitment's leaves.

Some users of this library run where device allocation is not theirs to make (memory reserved up front
by a serving loop, pools owned by an embedding process).  For them the library keeps the column hash's
scratch in a fixed in-library array; this test calls that entry point through the C ABI twice in a row,
on different shapes and keys, and requires the leaves of the ordinary allocating path bit for bit
(integer work: no tolerance).  The second call runs over the first call's leftovers in the shared array.
This file is collected last so that a failure here cannot hide any other test's result.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
P = 0xFFFFFFFF00000001


def _words(seed, n):
    i = np.arange(1, n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + i * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z % np.uint64(P)


def test_static_scratch_column_hash_matches_the_commit_path_twice_in_a_row():
    import torch
    from intelligenceregulation_b200 import backend

    dev = backend.B200Backend()
    torch.cuda.set_device(0)
    key = bytes(range(32))
    # (log_cols, inv_rate, rows, key): many chunks per column, then a ragged last chunk with another key rule
    calls = [(10, 4, 1100, key), (8, 4, 129, None), (6, 8, 5, key)]
    stores = []
    for si, (log_cols, ir, rows, k) in enumerate(calls):
        got = dev.try_commit(log_cols, ir, _words(77 + si, rows << log_cols), 16, k)
        assert got is not None, dev.ctx.declines
        stores.append(got)
    outs = []
    for (log_cols, ir, rows, k), (store, _) in zip(calls, stores):  # back to back, no sync in between
        out = torch.zeros(store.nn * 32, dtype=torch.uint8, device="cuda")
        backend.hash_columns_static(store.encoded_dev(), rows, store.nn, k, out.data_ptr(), torch.cuda.current_stream().cuda_stream)
        outs.append(out)
    torch.cuda.synchronize()
    for (store, leaves), out in zip(stores, outs):
        assert (out.cpu().numpy().reshape(store.nn, 32) == leaves).all()
    # a shape beyond the static array is refused, not attempted
    with pytest.raises(backend.DeviceError):
        backend.hash_columns_static(stores[0][0].encoded_dev(), 128 * 1000, 1 << 15, None, outs[0].data_ptr(), 0)
    for store, _ in stores:
        store.free()
    dev.ctx.close()
