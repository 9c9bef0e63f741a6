"""A seeded activation-lookup instance with the shapes of accuracy_act.rs: `groups` tables of 4096 words (word 2048 zero), queries on
rows of f_pad words of which `tokens` x `hidden` are live, mostly hits, some misses and out-of-range gates."""
import numpy as np


def instance(seed, groups, f_pad, rows, tokens, hidden, miss_every=37):
    rng = np.random.default_rng(seed)
    tables = rng.integers(-(1 << 20), 1 << 20, size=(groups, 4096), dtype=np.int64)
    tables[:, 2048] = 0
    ids = rng.integers(0, groups, size=hidden, dtype=np.uint32)
    n = rows * f_pad
    gates = rng.integers(-2048, 2048, size=n, dtype=np.int64)
    idx = np.arange(n)
    live = (idx // f_pad < tokens) & (idx % f_pad < hidden)
    grp = np.where(live, ids[np.minimum(idx % f_pad, hidden - 1)] if hidden else 0, 0)
    outputs = tables[grp, gates + 2048].copy()
    outputs[::miss_every] += 1                      # a wrong output: a miss
    gates[5::101] = 2048                            # key out of range: a miss
    gates[7::103] = -(1 << 40)                      # a forged gate: formed in the field, never wrapped
    return tables, ids, gates, outputs
