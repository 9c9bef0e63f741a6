"""Witness weight products on the device == matmul_reference (witness.rs:979-991, restated in oracle/witness.c), word for
word in int64: both weight layouts, strided activation and result planes with the untouched words zero, ragged shapes,
the int16 extremes that sit at the int32 accumulator bound (metal.rs:4234), the split over K; and the declines
(metal.rs:4662-4676): an activation outside int16, shapes outside the bounds.  Integer work: bit-exact."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from intelligenceregulation_b200 import backend

    c = backend.Context(0)
    yield c
    c.close()


def _case(seed, t, k, n, xs, os_, extreme=False):
    rng = np.random.default_rng(seed)
    x = rng.integers(-32768, 32768, size=(t - 1) * xs + k + 3, dtype=np.int64)
    w = rng.integers(-128, 128, size=k * n + 5, dtype=np.int8)
    if extreme:  # rows and columns of constant extremes: every partial sum at its largest magnitude, no cancellation
        x[:] = np.where(rng.integers(0, 2, x.size) == 1, 32767, -32768)
        for r, v in enumerate((255, 32767, -32768, -1, -256)):  # lo = 255 / hi = 127 / hi = -128 / (hi, lo) = (-1, 255) / (-1, 0)
            x[r * xs:r * xs + k] = v
        wm = np.where(rng.integers(0, 4, (n, k)) == 0, 127, -128).astype(np.int8)
        wm[0], wm[1] = -128, 127
        w[:k * n] = wm.reshape(-1)
    return x, w, (t - 1) * os_ + n + 2


@pytest.mark.parametrize("t,k,n,xs,os_,in_out", [
    (1, 1, 1, 1, 1, False), (3, 5, 7, 9, 11, True), (128, 64, 64, 64, 64, False), (128, 64, 64, 64, 64, True),
    (128, 4096, 1024, 4096, 1024, False), (128, 1024, 4096, 1024, 4096, True), (130, 200, 300, 210, 333, False),
    (257, 1000, 130, 1000, 130, True), (77, 4097, 65, 4100, 70, False), (16, 16400, 48, 16400, 48, False),
])
def test_product_equals_the_reference_words(ctx, oracle, t, k, n, xs, os_, in_out):
    x, w, out_len = _case(t * 31 + k, t, k, n, xs, os_)
    want = oracle.witness_product(t, x, xs, w, k, n, os_, out_len, in_out)
    got = ctx.witness_product(t, x, xs, w, k, n, os_, out_len, in_out)
    assert got is not None and (got == want).all()


@pytest.mark.parametrize("k", [4096, 65536])
def test_extremes_at_the_accumulator_bound(ctx, oracle, k):
    t, n = 8, 72
    x, w, out_len = _case(k, t, k, n, k, n, extreme=True)
    want = oracle.witness_product(t, x, k, w, k, n, n, out_len, False)
    got = ctx.witness_product(t, x, k, w, k, n, n, out_len, False)
    assert got is not None and (got == want).all()
    plane = want[:t * n].reshape(t, n)
    assert plane[0, 0] == -255 * 128 * k and plane[2, 0] == 32768 * 128 * k and plane[1, 1] == 32767 * 127 * k
    if k == 65536:  # the low-byte product of row 0 sits at the int32 bound; the plane's words need int64
        assert -(1 << 31) < plane[0, 0] < -(1 << 31) + (1 << 24) and plane[2, 0] > (1 << 37)


def test_declines(ctx, oracle):
    x, w, out_len = _case(1, 4, 64, 64, 64, 64)
    x[70] = 32768
    assert ctx.witness_product(4, x, 64, w, 64, 64, 64, out_len, False) is None   # an activation outside int16
    x[70] = -32769
    assert ctx.witness_product(4, x, 64, w, 64, 64, 64, out_len, False) is None
    x[70] = 5
    assert ctx.witness_product(4, x, 64, w, 64, 64, 64, out_len, False) is not None
    assert ctx.witness_product(4, x, 63, w, 64, 64, 64, out_len, False) is None   # xs < inner
    assert ctx.witness_product(4, x, 64, w, 64, 64, 60, out_len, False) is None   # os < outer
    assert ctx.witness_product(4, x, 64, w[:100], 64, 64, 64, out_len, False) is None  # weights too short
    assert ctx.witness_product(4, x, 64, w, 64, 64, 64, 100, False) is None       # rows outside the result plane
    assert ctx.witness_product(0, x, 64, w, 64, 64, 64, out_len, False) is None
    big = np.zeros(65537, dtype=np.int64)
    assert ctx.witness_product(1, big, 65537, np.zeros(65537, dtype=np.int8), 65537, 1, 1, 1, False) is None  # inner above 2^16


def test_resident_operands(ctx, oracle):
    import torch

    t, k, n = 128, 2048, 1536
    x, w, out_len = _case(9, t, k, n, k, n)
    d_x, d_w = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    d_out = torch.full((out_len,), 7, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    assert ctx.witness_product_dev(t, d_x.data_ptr(), x.size, k, d_w.data_ptr(), w.size, k, n, n, out_len, False, d_out.data_ptr())
    assert (d_out.cpu().numpy() == oracle.witness_product(t, x, k, w, k, n, n, out_len, False)).all()


@pytest.mark.parametrize("k,n", [(4096, 14336), (14336, 4096), (4096, 1024)])
def test_block_size_products_on_sampled_columns(ctx, oracle, k, n):
    """The 8B block's own shapes (T = 128): weights read in place, K split with atomics; the CPU restatement on three
    bands of output columns (the whole product would take it a minute)."""
    import torch

    t = 128
    g = torch.Generator().manual_seed(k + n)
    x = torch.randint(-32768, 32768, (t * k,), dtype=torch.int64, generator=g).numpy()
    w = torch.randint(-128, 128, (k * n,), dtype=torch.int8, generator=g).numpy()
    got = ctx.witness_product(t, x, k, w, k, n, n, t * n, False)
    assert got is not None
    got = got.reshape(t, n)
    for c0 in (0, (n // 2 // 64) * 64 + 13, n - 64):
        band = np.ascontiguousarray(w.reshape(n, k)[c0:c0 + 64])
        want = oracle.witness_product(t, x, k, band, k, 64, 64, t * 64, False).reshape(t, 64)
        assert (got[:, c0:c0 + 64] == want).all(), c0
    # linearity in the activations: W (x + x') = W x + W x' on the full plane (exact integers)
    x2 = torch.randint(-1000, 1000, (t * k,), dtype=torch.int64, generator=g).numpy()
    xs_ = np.clip(x, -30000, 30000)
    a = ctx.witness_product(t, xs_, k, w, k, n, n, t * n, False)
    b = ctx.witness_product(t, x2, k, w, k, n, n, t * n, False)
    c = ctx.witness_product(t, xs_ + x2, k, w, k, n, n, t * n, False)
    assert (a + b == c).all()
