"""Host logic of the device table builders, without a device: the index maps `plane_maps` makes (the host builder's own,
argument.rs:486-512), pushed through the kernels' formula in plain Python, give the words of the reference's walked
builder (oracle `priv_table`, argument.rs:386-577); the split eq cube equals the full one (argument.rs:586-660)."""
import numpy as np
import pytest

import tables_util as T


@pytest.mark.parametrize("case", [(1, 6, 0, 0, 1), (2, 6, 2, 0, 1), (3, 7, 3, 2, 3), (4, 5, 0, 2, 2), (5, 8, 1, 0, 1), (6, 1, 0, 0, 1), (7, 4, 4, 3, 1)])
def test_planned_maps_reproduce_the_walked_plane_table(oracle, case):
    from intelligenceregulation_b200 import backend

    seed, n_vars, n_fixed, n_unused, ns = case
    data = np.random.default_rng(seed).integers(0, T.P, size=1 << 13, dtype=np.uint64)
    coords, slices = T.random_plane(seed, n_vars, n_fixed, n_unused, ns, data.size)
    want = oracle.priv_table(coords, slices, data, n_vars)
    used, xlo, inv_lo, inv_hi, zbits, eqf = backend.plane_maps(n_vars, coords)

    def v(idx):
        a = (0, 0)
        for off, cf in slices:
            a = T.f2_add(a, T.f2_mul(cf, (int(data[off + idx]), 0)))
        return a

    for x in range(1 << n_vars):
        xu = x & used
        im = int(inv_hi[xu >> xlo]) | int(inv_lo[xu & ((1 << xlo) - 1)])
        if zbits.size == 0:
            got = v(im)
        else:
            got = (0, 0)
            for z in range(zbits.size):
                got = T.f2_add(got, T.f2_mul((int(eqf[z][0]), int(eqf[z][1])), v(im | int(zbits[z]))))
        assert got == (int(want[x][0]), int(want[x][1])), (case, x)


def test_a_variable_read_twice_is_not_planned():
    from intelligenceregulation_b200 import backend

    with pytest.raises(ValueError):
        backend.plane_maps(3, [("rho", 1), ("flip", 1)])


@pytest.mark.parametrize("case", [(5, 0, 5), (9, 2, 4), (9, 0, 9), (7, 6, 1), (6, 3, 0)])
def test_split_eq_cube_equals_the_full_cube(oracle, case):
    from intelligenceregulation_b200 import backend

    n_vars, start, p = case
    point = oracle.ZkRng(n_vars * 100 + p, b"eq").fp2_vec(max(p, 1))[:p]
    want = oracle.eq_cube(point, n_vars, start)
    p_lo = p // 2
    hi, lo = backend.eq_table_msb(point[: p - p_lo]), backend.eq_table_msb(point[p - p_lo:])
    assert (hi == oracle.eq_table_msb(point[: p - p_lo])).all() and (lo == oracle.eq_table_msb(point[p - p_lo:])).all()
    shift = n_vars - start - p
    for x in range(1 << n_vars):
        y = (x >> shift) & ((1 << p) - 1)
        a, b = hi[y >> p_lo], lo[y & ((1 << p_lo) - 1)]
        assert T.f2_mul((int(a[0]), int(a[1])), (int(b[0]), int(b[1]))) == (int(want[x][0]), int(want[x][1]))
