"""Shared by the table-builder tests: seeded plane descriptors in the reference's grammar (argument.rs `Priv`:
coordinates Rho / Flip / Fixed, slices)."""
import numpy as np

P = 0xFFFFFFFF00000001


def random_plane(seed, n_vars, n_fixed, n_unused, ns, data_words):
    """coords (first = most significant plane-index bit), slices, for a plane that reads n_vars - n_unused cube variables
    (each once, some flipped) and has n_fixed coordinates fixed at challenge points, in a shuffled order."""
    rng = np.random.default_rng(seed)
    vars_read = sorted(rng.choice(n_vars, size=n_vars - n_unused, replace=False).tolist())
    coords = [("flip" if rng.integers(0, 3) == 0 else "rho", int(k)) for k in vars_read]
    coords += [("fixed", (int(rng.integers(0, P, dtype=np.uint64)), int(rng.integers(0, P, dtype=np.uint64)))) for _ in range(n_fixed)]
    order = rng.permutation(len(coords))
    coords = [coords[i] for i in order]
    log = len(coords)
    assert data_words >= (1 << log)
    if ns == 1:
        slices = [(int(rng.integers(0, data_words - (1 << log) + 1)), (1, 0))]
    else:
        slices = [(int(rng.integers(0, data_words - (1 << log) + 1)),
                   (int(rng.integers(0, P, dtype=np.uint64)), int(rng.integers(0, P, dtype=np.uint64)) if s % 2 else 0)) for s in range(ns)]
    return coords, slices


def f2_add(a, b):
    return ((a[0] + b[0]) % P, (a[1] + b[1]) % P)


def f2_mul(a, b):
    return ((a[0] * b[0] + 7 * a[1] * b[1]) % P, (a[0] * b[1] + a[1] * b[0]) % P)
