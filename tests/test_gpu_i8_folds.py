"""int8 weight folds (zkp-core/src/mle.rs:157-319) on the device == the CPU restatement, for the shapes that take the 16-byte-load
kernel (whole 16-byte groups per row) and those that do not; values at the int8 extremes.  Field words: bit-exact."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from intelligenceregulation_b200 import backend

    c = backend.Context(0)
    yield c
    c.close()


@pytest.mark.parametrize("rows,cols", [(1, 512), (5, 528), (9, 4112), (8, 2048), (17, 6160), (3, 500), (4, 520), (64, 14336), (33, 40000)])
def test_fold_cols(ctx, oracle, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    m = rng.integers(-128, 128, size=(rows, cols), dtype=np.int8)
    m[0, :] = -128
    if rows > 1:
        m[1, :] = 127
    c = oracle.ZkRng(cols, b"i8-fold").fp2_vec(cols)
    c[::97] = np.array([0xFFFFFFFF00000000, 0xFFFFFFFF00000000], dtype=np.uint64)  # p - 1: the largest halves
    assert (ctx.fold_cols_i8(m, c) == oracle.fold_cols_i8(m, c)).all()


def test_fold_cols_block_shape(ctx, oracle):
    rng = np.random.default_rng(3)
    m = rng.integers(-128, 128, size=(4096, 14336), dtype=np.int8)
    c = oracle.ZkRng(5, b"i8-fold").fp2_vec(14336)
    got = ctx.fold_cols_i8(m, c)
    for r0 in (0, 2000, 4088):
        assert (got[r0:r0 + 8] == oracle.fold_cols_i8(m[r0:r0 + 8], c)).all()


@pytest.mark.parametrize("rows,cols", [(1, 8), (100, 64), (255, 4096), (256, 8), (257, 24), (1000, 520), (4096, 1030), (2049, 4096), (300, 6)])
def test_fold_rows(ctx, oracle, rows, cols):
    rng = np.random.default_rng(rows * 3 + cols)
    m = rng.integers(-128, 128, size=(rows, cols), dtype=np.int8)
    m[:, 0] = -128
    if cols > 1:
        m[:, 1] = 127
    w = oracle.ZkRng(rows, b"i8-fold-rows").fp2_vec(rows)
    w[::53] = np.array([0xFFFFFFFF00000000, 0xFFFFFFFF00000000], dtype=np.uint64)
    assert (ctx.fold_rows_i8(m, w) == oracle.fold_rows_i8(m, w)).all()


def test_fold_rows_block_shape(ctx, oracle):
    rng = np.random.default_rng(4)
    m = rng.integers(-128, 128, size=(14336, 4096), dtype=np.int8)
    w = oracle.ZkRng(6, b"i8-fold-rows").fp2_vec(14336)
    got = ctx.fold_rows_i8(m, w)
    for c0 in (0, 2048, 4032):
        assert (got[c0:c0 + 64] == oracle.fold_rows_i8(np.ascontiguousarray(m[:, c0:c0 + 64]), w)).all()
