"""Host side of the narrow witness upload: the width classes and the row packer mirror the reference's CUDA uploader
(hashline/src/gpu/cuda.rs:903-960 `narrow_class`, `pack_narrow`); widening the packed bytes restores every word."""
import numpy as np

P = 0xFFFFFFFF00000001


def widen(packed, widths, n):
    """`k_widen` (hashline/src/gpu/kernels.cu:227-236) in numpy"""
    out, at = [], 0
    for w in widths:
        w = int(w)
        raw = packed[at:at + w * n]
        at += w * n
        if w == 8:
            out.append(raw.view(np.uint64))
            continue
        x = raw.view({1: np.int8, 2: "<i2", 4: "<i4"}[w]).astype(np.int64)
        out.append(np.where(x >= 0, x.astype(np.uint64), (x + (1 << 32)).astype(np.uint64) + np.uint64(P - (1 << 32))))
    assert at == packed.size
    return np.concatenate(out)


def test_width_classes_at_their_boundaries():
    from intelligenceregulation_b200 import backend

    cls = lambda *v: backend.narrow_class(np.array(v, dtype=np.uint64))  # noqa: E731
    assert cls(0, 127, P - 128, P - 1) == 1
    assert cls(128) == 2 and cls(P - 129) == 2 and cls(0x7FFF, P - 0x8000) == 2
    assert cls(0x8000) == 4 and cls(P - 0x8001) == 4 and cls(0x7FFFFFFF, P - 0x80000000) == 4
    assert cls(0x80000000) == 8 and cls(P - 0x80000001) == 8 and cls(1 << 40) == 8


def test_pack_rows_round_trips_every_word():
    from intelligenceregulation_b200 import backend

    rng = np.random.default_rng(3)
    n = 64
    to_fp = lambda v: np.where(v >= 0, v.astype(np.uint64), (v + (1 << 32)).astype(np.uint64) + np.uint64(P - (1 << 32)))  # noqa: E731
    rows = [to_fp(rng.integers(-128, 128, n)), to_fp(rng.integers(-32768, 32768, n)), to_fp(rng.integers(-(1 << 31), 1 << 31, n)),
            rng.integers(0, P, n, dtype=np.uint64), to_fp(np.array([-128, 127, -1, 0] * 16)), to_fp(np.array([-32768, 32767, 128, -129] * 16)),
            to_fp(np.array([-(1 << 31), (1 << 31) - 1, 32768, -32769] * 16)), np.array([P - 1, 0, 1 << 31, P - (1 << 31) - 1] * 16, dtype=np.uint64)]
    data = np.concatenate(rows)
    packed, widths = backend.pack_rows(data, len(rows))
    assert list(widths) == [1, 2, 4, 8, 1, 2, 4, 8]
    assert packed.size == sum(int(w) for w in widths) * n
    assert (widen(packed, widths, n) == data).all()
