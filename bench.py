"""Ligero-commit throughput of the B200 backend (and of the CPU restatement beside it).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = one hiding commitment of one transformer block's `A` matrix at the Llama-3-8B block
shape the reference registers (W16R2_8B_T128_H24: 2,504 rows x 2^14 -> 2^15 columns, Q = 280 pads
per row, keyed column hash), through to its salted Merkle root: inverse NTT, pad + coset scaling,
forward NTT, BLAKE3 column leaves, salted leaves, tree.  Metric: encoded bytes (rows * nn * 8)
per second, the reference's own accounting for "commit GB/s".

The witness is what a block's `A` matrix holds: int16-valued words (seeded, uniform) in all but eight rows, which carry
full-width field words (the rows a prover fills with digests and masks).
`value`  - inputs already resident in HBM, timed with CUDA events on the library's stream.
`e2e`    - the same commitment through the host-pointer C-ABI call a prover makes (hl_b200_commit_zk_packed: the witness
           rows travel as their narrow bytes, as the reference's CUDA uploader sends them, and are widened on the device),
           page-locked host inputs, H2D and D2H inside the clock.
With N > 1 every rank commits its own blocks (D55 sharding: block k belongs to rank k mod N; no
data-path collective) and the 32-byte roots are all-gathered over NCCL, as the join needs them.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORK = {"log_cols": 14, "inv_rate": 2, "q": 280, "rows": 2504, "profile": "hashline-zk-mr1/b200-bench/1"}
P = 0xFFFFFFFF00000001
WIDE_ROW_STEP = 313  # every 313th row of the witness holds full-width words (8 of 2,504)


def encode_dram_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the encoder at this workload, from the committed record of
    the ncu capture (with its command) beside the text summary of the same capture; None when the record is absent."""
    try:
        rec = json.load(open(os.path.join(ROOT, "profiles", "k_encode_fast_8b_A.json")))
        return int(rec["dram_bytes_read"]) + int(rec["dram_bytes_write"])
    except (OSError, KeyError, ValueError):
        return None

PUBLISHED_GBPS = 26.0  # the reference's own published figure: its Metal backend on an M3 Ultra at this exact shape


def splitmix_fp(seed: int, n: int) -> np.ndarray:
    """Seeded uniform field elements: SplitMix64 words reduced mod p (the generator of the reference's
    encode vectors, zkp-core/src/pcs/encode_conformance_tests.rs:28-47)."""
    i = np.arange(1, n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + i * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z % np.uint64(P)


def witness_words(seed: int, rows: int, n: int) -> np.ndarray:
    """The block's `A` rows: int16-valued field words (x >= 0 as x, x < 0 as p + x), every WIDE_ROW_STEP-th row full-width."""
    v = (splitmix_fp(seed, rows * n) % np.uint64(65536)).astype(np.int64) - 32768
    out = np.where(v >= 0, v.astype(np.uint64), (v + (1 << 32)).astype(np.uint64) + np.uint64(P - (1 << 32))).reshape(rows, n)
    wide = np.arange(0, rows, WIDE_ROW_STEP)
    out[wide] = splitmix_fp(seed ^ 0x5A5A, wide.size * n).reshape(wide.size, n)
    return out.reshape(-1)


def block_inputs(block: int):
    """seeded inputs of one block's commitment: (data, pads, salts) as the prover would hold them"""
    import blake3 as b3

    w = WORK
    n, nn = 1 << w["log_cols"], (1 << w["log_cols"]) * w["inv_rate"]
    data = witness_words(0xB2000100 + block, w["rows"], n)
    pads = splitmix_fp(0xB2000200 + block, w["rows"] * w["q"])
    salts = np.frombuffer(b3.blake3(b"bench-salts-%d" % block).digest(length=nn * 32), dtype=np.uint8).copy()
    return data, pads, salts


def coset_powers(nn: int) -> np.ndarray:
    out, x = np.empty(nn, dtype=np.uint64), 1
    for i in range(nn):
        out[i] = x
        x = x * 7 % P
    return out


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_indices):
        self.idx, self.rows, self.proc = ",".join(str(i) for i in gpu_indices), [], None

    def start(self):
        if not self.idx:
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", self.idx],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.t.join(timeout=2)
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) < 9:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_commit(o, data, pads, salts):
    """One hiding commitment of the whole workload matrix on the host cores (the CPU restatement of pcs.rs:782-817): encode,
    keyed column hash, salted leaves, tree.  Returns (seconds, root)."""
    w = WORK
    n, nn, q, rows = 1 << w["log_cols"], (1 << w["log_cols"]) * w["inv_rate"], w["q"], w["rows"]
    tag = o.HashTag.for_profile(w["profile"])
    pows = o.coset_powers(7, nn)
    t0 = time.perf_counter()
    enc = o.encode_rows_zk(data, rows, n, pads, q, pows, w["log_cols"] + 1)
    leaves = o.hash_columns(enc, rows, nn, tag.column)
    levels = o.merkle_build(o.salt_leaves(leaves, salts.reshape(nn, 32), tag.leaf), tag.node)
    return time.perf_counter() - t0, bytes(levels[-1])


CPU_NOTE = ("all {rows} rows per step, the same seeded matrix the GPU arm commits: encode + keyed column hash + salt + tree; C restatement "
            "(OpenMP, scalar BLAKE3 compiled for x86-64-v2) of the reference's Rust CPU path, which cannot be built in this image "
            "(no cargo); the reference's own CPU hashes with the blake3 crate's SIMD code, so this baseline is slower than the reference's would be")


def run_reference(args, rank: int) -> None:
    """The reference arm: the prover's CPU path on this box's host cores, on the whole workload matrix of block 0.  The
    reference's own binary is Rust and cannot be built here (no cargo in this image), so this times the C restatement of it
    (oracle/, OpenMP over rows / column tiles, the reference's task grains) and says so."""
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import hl_oracle as o

    if "LOCAL_RANK" in os.environ:  # torchrun pins OMP_NUM_THREADS=1 for its workers; this arm is the only worker that computes
        o.set_threads(len(os.sched_getaffinity(0)))
    w = WORK
    nn = (1 << w["log_cols"]) * w["inv_rate"]
    data, pads, salts = block_inputs(0)
    root = b""
    for _ in range(args.warmup):
        cpu_commit(o, data, pads, salts)
    t = []
    for _ in range(args.steps):
        sec, root = cpu_commit(o, data, pads, salts)
        t.append(sec)
    sec = sum(t) / len(t)
    gbps = w["rows"] * nn * 8 / sec / 1e9
    cores = o.num_threads()
    line = {
        "impl": "reference", "metric": "ligero_commit_GBps", "value": gbps, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64",
        "data": "synthetic", "config": workload_config(1),
        "cpu_baseline": {"value": gbps, "unit": "GB/s", "cores": cores, "kind": "port", "sample": CPU_NOTE.format(rows=w["rows"])},
        "e2e": {"value": gbps, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "root": root.hex(),
    }
    print(json.dumps(line))


def workload_config(world: int) -> dict:
    w = WORK
    return {"workload": "Ligero hiding commit of the Llama-3-8B block's A matrix (W16R2_8B_T128_H24): "
                        f"{w['rows']} rows x 2^{w['log_cols']} -> 2^{w['log_cols'] + 1} (rate 1/2), Q = {w['q']}, keyed BLAKE3 leaves, salted tree to the root",
            "rows": w["rows"], "log_cols": w["log_cols"], "inv_rate": w["inv_rate"], "q_pad": w["q"],
            "witness": f"int16-valued words (seeded uniform), every {WIDE_ROW_STEP}th row full-width field words; pads and salts seeded",
            "parallelism": f"d55-block-sharding x{world}" if world > 1 else "single",
            "l2": "inputs (328 MB) and encoding (656 MB) exceed the 126 MB L2; no flush needed",
            "published_baseline": "26.0 GB/s, reference Metal backend on Apple M3 Ultra, same shape"}


def structured_rhos(dense: np.ndarray) -> np.ndarray:
    k, rows, _ = dense.shape
    out = np.zeros_like(dense)
    out[k - 1] = dense[k - 1]
    for g in range(k - 1):
        r0 = (g * 64) % (rows - 40)
        out[g, r0:r0 + 32] = dense[g, r0:r0 + 32]
        out[g, rows - 3:rows - 1] = dense[g, rows - 3:rows - 1]
    return out


def device_extras(dev, backend, np_data, np_pads, np_pows, col_key, only: str = "") -> dict:
    """Device time (CUDA events inside the library, per kernel family) of the rest of one block's device work at the
    same shape: the opening of `A` (38 row combinations with pads, 280 gathered columns), a 2^21-point degree-3
    zero-check sumcheck batch (the LogUp query side), the LogUp helper column of 2^21 queries, and one FFN weight fold."""
    w = WORK
    log_cols, ir, q, rows = w["log_cols"], w["inv_rate"], w["q"], w["rows"]
    ctx = dev.ctx
    out = {}
    import torch

    def want(name):  # --only a,b,c limits the run to those families (a profiler capture of one kernel family)
        return not only or name in only.split(",")

    rhos = splitmix_fp(77, 38 * rows * 2).reshape(38, rows, 2)
    ctx.timing_read(reset=True)
    ctx.timing_enable(True)
    if want("open"):
        st, _ = dev.try_commit_zk_keyed(log_cols, ir, np_data, np_pads, np_pows, log_cols + 1, col_key)
        idx = (splitmix_fp(78, 280) % np.uint64(st.nn)).astype(np.uint64)
        for _ in range(2):
            st.fold_rows_with_pads(rhos)
            st.columns(idx)
        ctx.timing_read(reset=True)
        ctx.timing_enable(True)
        for _ in range(3):
            st.fold_rows_with_pads(rhos)
            st.columns(idx)
        t = ctx.timing_read(reset=True)
        out["open_A_fold_38rho_ms"] = t["fold"][0] / 3
        out["open_A_gather_280cols_ms"] = t["gather"][0] / 3
        # the shape of a real opening (pcs.rs:851-891, 952-973): 37 group vectors that live on their claim's 32 plane rows and
        # the two mask rows, one dense proximity vector; the dense figure above is the worst case
        srho = structured_rhos(rhos)
        for _ in range(2):
            st.fold_rows_with_pads(srho)
        ctx.timing_read(reset=True)
        for _ in range(3):
            st.fold_rows_with_pads(srho)
        out["open_A_fold_37_plane_vectors_1_dense_ms"] = ctx.timing_read(reset=True)["fold"][0] / 3
        st.free()
    if want("sumcheck"):
        n = 21
        tables = splitmix_fp(79, 3 * (1 << n) * 2).reshape(3, 1 << n, 2)
        alpha = splitmix_fp(80, 2).reshape(1, 2)
        mask = splitmix_fp(81, ((n + 1) * 3 + 2) * 2).reshape(-1, 2)
        for rep in range(3):
            ev = backend.B200Rounds(ctx, backend.POLY_LOGUP_Q, tables, 3, alpha)
            if rep == 1:
                ctx.timing_read(reset=True)
            ev.batched(n, bytes(32), 0, None, mask=mask, mask_vars=n + 1, mask_c=(3, 5), recover_one=True, claim=(0, 0))
            ev.free()
        t = ctx.timing_read(reset=True)
        out["sumcheck_logup_q_2^21_deg3_21rounds_ms"] = t["rounds"][0] / 2
        ctx.set_dependent_launch(False)  # the same batch with every kernel an ordinary stream launch
        for rep in range(3):
            ev = backend.B200Rounds(ctx, backend.POLY_LOGUP_Q, tables, 3, alpha)
            if rep == 1:
                ctx.timing_read(reset=True)
            ev.batched(n, bytes(32), 0, None, mask=mask, mask_vars=n + 1, mask_c=(3, 5), recover_one=True, claim=(0, 0))
            ev.free()
        out["sumcheck_logup_q_2^21_deg3_21rounds_plain_launches_ms"] = ctx.timing_read(reset=True)["rounds"][0] / 2
        ctx.set_dependent_launch(True)
    if want("helpers"):
        nq = 1 << 21
        qidx = (splitmix_fp(82, nq) % np.uint64(1 << 16)).astype(np.int32)
        qout = (splitmix_fp(83, nq) % np.uint64(1 << 15)).astype(np.int32)
        for rep in range(3):
            if rep == 1:
                ctx.timing_read(reset=True)
            ctx.logup_helpers(qidx, qout, (11, 12), (13, 14), (15, 16))
        t = ctx.timing_read(reset=True)
        out["logup_helpers_2^21_ms"] = t["logup"][0] / 2
    if want("i8folds"):
        wm = (splitmix_fp(84, 4096 * 14336) % np.uint64(256)).astype(np.uint8).view(np.int8).reshape(4096, 14336)
        cw = splitmix_fp(85, 14336 * 2).reshape(14336, 2)
        for rep in range(3):
            if rep == 1:
                ctx.timing_read(reset=True)
            ctx.fold_cols_i8(wm, cw)
        t = ctx.timing_read(reset=True)
        out["fold_cols_i8_4096x14336_ms"] = t["fold"][0] / 2
        rw = splitmix_fp(89, 4096 * 2).reshape(4096, 2)
        for rep in range(3):
            if rep == 1:
                ctx.timing_read(reset=True)
            ctx.fold_rows_i8(wm, rw)
        out["fold_rows_i8_4096x14336_ms"] = ctx.timing_read(reset=True)["fold"][0] / 2
    if want("rng"):
        # the pads and salts of the hiding commitment of `A` expanded on the device from the caller's generator key
        # (rows * q field draws, then nn salts of four words: 11.2 MB + 1 MB of BLAKE3 extended output)

        d_rng = torch.empty(rows * q + 4 * ((1 << log_cols) * ir), dtype=torch.int64, device="cuda")
        nn_ = (1 << log_cols) * ir
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cs = torch.cuda.current_stream()
        for rep in range(3):
            if rep == 1:
                ev0.record(cs)
            ctx.rng_fill_dev(bytes(range(32)), 0, rows * q, True, d_rng.data_ptr())
            ctx.rng_fill_dev(bytes(range(32)), 2 * rows * q, 4 * nn_, False, d_rng.data_ptr() + 8 * rows * q)
        ev1.record(cs)
        torch.cuda.synchronize()
        out["draw_pads_and_salts_of_A_ms"] = ev0.elapsed_time(ev1) / 2
        del d_rng
    if want("lookup"):
        # the helper half of H for the byte-table lookups (protocol.rs:1700-1800): one job = 2^25 looked word pairs, two
        # 256-entry inverse tables, two planes written (2 x 8 B read, 2 x 8 B written per pair)
        npair = 1 << 25
        d_a = torch.from_numpy((splitmix_fp(92, npair) % np.uint64(256)).astype(np.int64)).cuda()
        d_b = torch.from_numpy((splitmix_fp(93, npair) % np.uint64(256)).astype(np.int64)).cuda()
        d_t = torch.empty(1024, dtype=torch.int64, device="cuda")
        d_h = torch.empty(2 * npair, dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        for rep in range(3):
            if rep == 1:
                ctx.timing_read(reset=True)
            ctx.lookup_inverse_table((21, 22), (23, 24), 8, d_t.data_ptr())
            ctx.lookup_inverse_table((21, 22), (25, 26), 8, d_t.data_ptr() + 4096)
            ctx.lookup_helpers_dev(d_a.data_ptr(), d_t.data_ptr(), 8, (23, 24), (21, 22), npair, d_h.data_ptr(), d_h.data_ptr() + 8 * npair,
                                   d_b=d_b.data_ptr(), d_table_b=d_t.data_ptr() + 4096, log_b=8, g_b=(25, 26))
        out["lookup_helpers_u8_pairs_2^25_ms"] = ctx.timing_read(reset=True)["logup"][0] / 2
        del d_a, d_b, d_t, d_h
    if want("slots"):
        # a slot's tables built on the device from the resident rows of `A`: an eq cube of 2^21 entries and a witness plane of
        # 2^19 entries partially evaluated at 3 fixed coordinates (8 rows of 2^14 words each folded per entry)
        st, _ = dev.try_commit_zk_keyed(log_cols, ir, np_data, np_pads, np_pows, log_cols + 1, col_key)
        point = splitmix_fp(90, 21 * 2).reshape(21, 2)
        coords = [("fixed", (int(a), int(b))) for a, b in splitmix_fp(91, 6).reshape(3, 2)] + [("rho", k) for k in range(19)]
        for rep in range(3):
            if rep == 1:
                ctx.timing_read(reset=True)
            t21, t19 = backend.B200Tables(ctx, 1, 21), backend.B200Tables(ctx, 1, 19)
            t21.plan_eq(0, point, 0)
            t19.plan_plane(0, st, coords, [(0, (1, 0))])
            t21.flush(); t19.flush()
            t21.free(); t19.free()
        t = ctx.timing_read(reset=True)
        out["tables_eq_2^21_plus_plane_2^19_x8_ms"] = t["tables"][0] / 2
        m125 = _m125_replay_slots(backend.SlotProgram)
        note125 = "the reference's recorded 125M slot graphs (T512 / d768 / f2048) at their recorded sizes: 23 slots, 258 tables, cubes of 2^8 .. 2^22 points"
        slot_replay(dev, backend, st, rows, 1 << log_cols, m125, note125)  # warm-up: first launches size the device's local-memory pool
        out["slot_replay"] = slot_replay(dev, backend, st, rows, 1 << log_cols, m125, note125)
        w16 = _w16r2_slots(backend.SlotProgram)
        note8b = ("the slot graphs of a real W16R2 block core (recorded coefficient values) at the cube sizes of the Llama-3-8B block shape "
                  "W16R2_8B_T128_H24: 23 slots, 1.44 GB of tables")
        slot_replay(dev, backend, st, rows, 1 << log_cols, w16, note8b)
        out["slot_replay_8B_T128"] = slot_replay(dev, backend, st, rows, 1 << log_cols, w16, note8b)
        # the opening of `H` (10 row combinations: the proximity vector and nine that live on a plane's rows) on this store as a stand-in
        hrho = structured_rhos(rhos[:10])
        for rep in range(3):
            if rep == 1:
                ctx.timing_read(reset=True)
            st.fold_rows_with_pads(hrho)
        out["open_H_fold_9_plane_vectors_1_dense_ms"] = ctx.timing_read(reset=True)["fold"][0] / 2
        st.free()
    if want("slot_program"):
        # the heaviest slot polynomial of a block as data: the recorded structure of the D zero-check (60 tables, 71 nodes,
        # declared degree 5) with seeded coefficients, at 2^19 points (the 8B block domain of this slot: 128 tokens x width 4096), through the interpreting evaluator
        prog, deg, base = slot14_program(backend.SlotProgram)
        n = 19
        tables = slot14_tables(prog, base, n)
        mask = splitmix_fp(88, ((n + 1) * deg + 2) * 2).reshape(-1, 2)
        for rep in range(3):
            ev = backend.B200Rounds(ctx, prog, tables, deg)
            if rep == 1:
                ctx.timing_read(reset=True)
            ev.batched(n, bytes(32), 0, None, mask=mask, mask_vars=n + 1, mask_c=(3, 5), recover_one=True, claim=(0, 0))
            ev.free()
        t = ctx.timing_read(reset=True)
        out["sumcheck_slot_program_60tables_71nodes_deg5_2^19_ms"] = t["rounds"][0] / 2
    if want("mask"):
        # the masking commitment M of a block (zk.rs:447-656): 24 masks -> 48 message rows of 512 + 4 rows of 1024 coefficients
        # on the coset of 4096, column hashes, salted tree; then the opening's product polynomial, proximity fold, 256 columns
        S = 24
        mm = splitmix_fp(94, 2 * S * 512).reshape(2 * S, 512)
        mm[:, 320:] = 0
        mcoef, mpows = splitmix_fp(95, 4 * 1024).reshape(4, 1024), coset_powers(4096)
        msalts = splitmix_fp(96, 4096 * 4).view(np.uint8).reshape(4096, 32)
        mws, mrs = splitmix_fp(97, S * 512 * 2).reshape(S, 512, 2), splitmix_fp(98, (2 * S + 2) * 2).reshape(-1, 2)
        midx = (splitmix_fp(99, 256) % np.uint64(4096)).astype(np.uint64)
        t_c = t_o = 0.0
        for rep in range(4):
            t0 = time.perf_counter()
            dm = backend.mask_commit(ctx, mm, mcoef, mpows, col_key)
            dm.merkle(msalts, col_key, col_key)
            t1 = time.perf_counter()
            dm.open_q(mws); dm.prox(mrs); dm.columns(midx)
            t2 = time.perf_counter()
            dm.free()
            if rep:
                t_c, t_o = t_c + (t1 - t0) * 1e3 / 3, t_o + (t2 - t1) * 1e3 / 3
        out["mask_M_24masks_commit_and_tree_wall_ms"] = t_c  # host wall time of the calls: uploads, launches, read-backs
        out["mask_M_24masks_open_wall_ms"] = t_o
    if want("witness"):
        # the witness weight products of one 8B block at T = 128 (witness.rs:818-835): q, k, v, o, gate, up, down with the
        # weights resident; int16 activations, int8 weights, exact int64 planes
        wp_shapes = [("q", 4096, 4096), ("k", 4096, 1024), ("v", 4096, 1024), ("o", 4096, 4096), ("gate", 4096, 14336), ("up", 4096, 14336), ("down", 14336, 4096)]
        gw = torch.Generator(device="cuda").manual_seed(5)
        d_wmax = torch.randint(-128, 128, (4096 * 14336,), dtype=torch.int8, device="cuda", generator=gw)
        d_xw = torch.randint(-32768, 32768, (128 * 14336,), dtype=torch.int64, device="cuda", generator=gw)
        d_ow = torch.empty(128 * 14336, dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        per, macs = {}, 0
        for name, kk, nn2 in wp_shapes:
            for rep in range(4):
                if rep == 1:
                    ctx.timing_read(reset=True)
                assert ctx.witness_product_dev(128, d_xw.data_ptr(), 128 * kk, kk, d_wmax.data_ptr(), kk * nn2, kk, nn2, nn2, 128 * nn2, False, d_ow.data_ptr())
            per[name] = round(ctx.timing_read(reset=True)["witness"][0] / 3, 4)
            macs += 128 * kk * nn2
        tot = sum(per.values())
        out["witness_products_8B_block_T128_ms"] = tot
        out["witness_products_detail"] = {"per_product_ms": per, "int8_TMAC_per_s": 2 * macs / (tot * 1e-3) / 1e12,
                                          "weight_bytes": sum(k_ * n_ for _, k_, n_ in wp_shapes),
                                          "weights_read_once_at_measured_hbm_ms": sum(k_ * n_ for _, k_, n_ in wp_shapes) / 6549.8e9 * 1e3}
        del d_wmax, d_xw, d_ow
    if want("long_rows"):
        # the T256 / T512 profiles (shape.rs:248-262): the same 41 M words as rows of 2^15 and 2^16, which run as 2 or 4
        # shared-memory transforms of 2^14 each way
        for lc, rws in ((15, rows // 2), (16, rows // 4)):
            nnl = (1 << lc) * ir
            dd = torch.from_numpy(splitmix_fp(0xB2000300 + lc, rws << lc).view(np.int64)).cuda()
            dp = torch.from_numpy(splitmix_fp(0xB2000400 + lc, rws * q).view(np.int64)).cuda()
            dw = torch.from_numpy(coset_powers(nnl).view(np.int64)).cuda()
            torch.cuda.synchronize()
            for rep in range(4):
                if rep == 1:
                    ctx.timing_read(reset=True)
                stl = dev.commit_zk_dev(lc, ir, dd.data_ptr(), rws, dp.data_ptr(), q, dw.data_ptr(), col_key)
                stl.free()
            t = ctx.timing_read(reset=True)
            out[f"commit_rows_of_2^{lc}_x{rws}_encode_ms"] = t["encode"][0] / 3
            out[f"commit_rows_of_2^{lc}_x{rws}_hash_ms"] = t["hash"][0] / 3
            del dd, dp, dw
    if want("commit_h"):
        # the helper commitment `H` of the block: 2,606 rows of 2^14 full-width words (the helper columns are field inverses), resident
        rows_h = 2606
        dd = torch.from_numpy(splitmix_fp(0xB2000500, rows_h << log_cols).view(np.int64)).cuda()
        dp = torch.from_numpy(splitmix_fp(0xB2000600, rows_h * q).view(np.int64)).cuda()
        dw = torch.from_numpy(coset_powers((1 << log_cols) * ir).view(np.int64)).cuda()
        dsalt = torch.zeros(((1 << log_cols) * ir) * 32, dtype=torch.uint8, device="cuda")
        dlev = torch.empty((2 * ((1 << log_cols) * ir) - 1) * 32, dtype=torch.uint8, device="cuda")
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cs = torch.cuda.current_stream()
        torch.cuda.synchronize()
        for rep in range(4):
            if rep == 1:
                ea.record(cs)
            sth = dev.commit_zk_dev(log_cols, ir, dd.data_ptr(), rows_h, dp.data_ptr(), q, dw.data_ptr(), col_key)
            sth.merkle_dev(dsalt.data_ptr(), col_key, col_key, dlev.data_ptr())
            sth.free()
        eb.record(cs)
        torch.cuda.synchronize()
        out["commit_H_2606x2^14_to_root_ms"] = ea.elapsed_time(eb) / 3
        del dd, dp, dw, dsalt, dlev
    if want("verify"):
        # the verifier's data-parallel part for one opening of `A` (pcs.rs:1282-1331): 39 clear vectors encoded (78 rows), 280 opened
        # columns hashed, walked to the root and combined with 39 row weights; host buffers in, verdicts out, wall time of the call
        vin = verifier_inputs(dev, np_data, np_pads, np_pows, col_key, rhos)
        for rep in range(4):
            if rep == 1:
                t0 = time.perf_counter()
            v = dev.check_opening_columns(log_cols, ir, np_pows, log_cols + 1, *vin["args"])
        out["verify_280_columns_39_vectors_wall_ms"] = (time.perf_counter() - t0) * 1e3 / 3
        assert v is not None and (v == 0).all(), "the verifier refused an honest opening"
        # the same call with its large inputs in page-locked memory (as the end-to-end commit leg has them)
        keep = []

        def pinned(a):
            t = torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1)).pin_memory()
            keep.append(t)
            return t.numpy().view(a.dtype).reshape(a.shape)

        pa = list(vin["args"])
        for j in (0, 3, 8, 9):  # columns, paths, row weights, clear vectors
            pa[j] = pinned(pa[j])
        for rep in range(4):
            if rep == 1:
                t0 = time.perf_counter()
            v = dev.check_opening_columns(log_cols, ir, np_pows, log_cols + 1, *pa)
        out["verify_280_columns_39_vectors_page_locked_wall_ms"] = (time.perf_counter() - t0) * 1e3 / 3
        assert v is not None and (v == 0).all(), "the verifier refused an honest opening"
    ctx.timing_enable(False)
    return out


def verifier_inputs(dev, np_data, np_pads, np_pows, col_key, rhos38) -> dict:
    """An honest opening of the bench's `A` commitment as the verifier receives it: 39 clear vectors, 280 opened columns with salts and paths."""
    w = WORK
    log_cols, ir, q, rows = w["log_cols"], w["inv_rate"], w["q"], w["rows"]
    nn = (1 << log_cols) * ir
    salts = (splitmix_fp(0xB2000700, nn * 4).view(np.uint8)).reshape(nn, 32)
    st, _, levels = dev.try_commit_zk_tree(log_cols, ir, np_data, np_pads, np_pows, log_cols + 1, col_key, salts, col_key, col_key, want_leaves=False)
    rhos = np.concatenate([structured_rhos(rhos38), splitmix_fp(0xB2000701, rows * 2).reshape(1, rows, 2)])
    vecs = st.fold_rows_with_pads(rhos)
    idx = (splitmix_fp(78, 280) % np.uint64(nn)).astype(np.uint64)
    cols = st.columns(idx)
    st.free()
    depth = log_cols + (ir.bit_length() - 1)
    paths = np.empty((280, depth, 32), dtype=np.uint8)
    for c, j in enumerate(idx):  # merkle.rs:92-100: the sibling at every level below the root
        off, width, i = 0, nn, int(j)
        for l in range(depth):
            paths[c, l] = levels[off + (i ^ 1)]
            off, width, i = off + width, width // 2, i >> 1
    return {"args": (cols, idx, np.ascontiguousarray(salts[idx.astype(np.int64)]), paths, bytes(levels[-1]), col_key, col_key, col_key, rhos, vecs),
            "levels": levels}


def _m125_slots():
    import json as _json

    return _json.load(open(os.path.join(ROOT, "intelligenceregulation_b200", "slot_graphs", "m125.json")))["slots"]


def _program_from_structure(SP, slot, coef):
    """a recorded slot graph (structure only) with coefficients drawn by class from `coef`"""
    prog = SP(len(slot["table_fields"]))

    def fw(f):
        return SP.node(f["n"]) if "n" in f else f["t"]

    for nd in slot["nodes"]:
        if "affine" in nd:
            prog.affine(coef("kbase") if nd["konst"] else "zero", [(coef(c), t) for c, t in nd["affine"]])
        else:
            prog.sum([(coef(c), [fw(f) for f in fs]) for c, fs in nd["sum"]])
    for t in slot["terms"]:
        prog.term(coef(t["coef"]), t["wrapper"], [fw(f) for f in t["inner"]])
    return prog


def slot14_program(SP):
    """the recorded structure of the D zero-check (60 tables, 71 nodes, declared degree 5) with seeded coefficients"""
    slot = _m125_slots()[14]
    cs = iter(splitmix_fp(86, 4096).tolist())

    def coef(cls):
        return "one" if cls == "one" else (next(cs) % (1 << 40), 0) if cls == "kbase" else (next(cs), next(cs))

    return _program_from_structure(SP, slot, coef), slot["declared_degree"], [f == "base" for f in slot["table_fields"]]


def slot14_tables(prog, base, nv):
    """seeded tables; the ones the reference records as base-valued (witness planes, public shape tables: 40 of 60) keep a
    zero imaginary word, as they do until the first fold"""
    t = splitmix_fp(87, prog.n_tables * (1 << nv) * 2).reshape(prog.n_tables, 1 << nv, 2)
    for i, b in enumerate(base):
        if b:
            t[i, :, 1] = 0
    return t


# main-round counts of the 23 slots at the Llama-3-8B block shape W16R2_8B_T128_H24 (T = 128, width 4096, hidden 14336, 32 query and
# 8 key-value heads of 128, rows of 2^14 words): shape.rs:2660-2714 `slots()` over the domain logs of shape.rs:2415-2451 with the
# lift of layout.rs:175-181 (T 7, L 14, D 19, Q 19, Kv 17, S 19, F 21, Tab 14; matmul inner axes 12, 12, 12, 10, 10, 12, 12, 12, 14)
SLOT_ROUNDS_8B = [19, 19, 7, 14, 19, 12, 12, 12, 10, 10, 12, 12, 12, 14, 19, 19, 17, 19, 21, 14, 14, 19, 19]
SLOT_NAMES = ["SS", "SSM", "TZC", "LZC", "RS", "QMM", "KMM", "VMM", "SCORE", "PV", "WO", "GMM", "UMM", "DMM", "DZC", "QZC", "KVZC", "SZC", "FZC", "TAB", "ZS",
              "IO_IN", "IO_OUT"]


def _w16r2_slots(SP):
    """[(name, main rounds at the 8B shape, degree, program, per-table kind)] from the slot graphs of a real W16R2 block core with
    their recorded coefficient values (intelligenceregulation_b200/slot_graphs/w16r2.json)"""
    import json as _json

    out = []
    for sl in _json.load(open(os.path.join(ROOT, "intelligenceregulation_b200", "slot_graphs", "w16r2.json")))["slots"]:
        prog = SP(len(sl["tables"]))

        def cv(c):
            return "one" if c[2] == "one" else "neg-one" if c[2] == "neg-one" else (c[0], c[1])

        def fw(f):
            return SP.node(f[1]) if f[0] == "n" else f[1]

        for nd in sl["nodes"]:
            if "affine" in nd:
                prog.affine((nd["konst"][0], nd["konst"][1]), [(cv(c), t) for c, t in nd["affine"]])
            else:
                prog.sum([(cv(c), [fw(f) for f in fs]) for c, fs in nd["sum"]])
        for t in sl["terms"]:
            prog.term(cv(t["coef"]), t["wrapper"], [fw(f) for f in t["inner"]])
        # witness planes, supports and endpoints are base-valued until the first fold; helper tables (h = re + u im) and, in the matmul
        # slots, the public folded weights are extension-valued from the start (the field kinds the reference records for these tables)
        matmul = 5 <= sl["slot"] <= 13
        kinds = ["eq" if k in ("eq", "geq") else "ext" if (k == "H" or (k == "pub" and matmul)) else "base" for k in sl["tables"]]
        out.append((SLOT_NAMES[sl["slot"]], SLOT_ROUNDS_8B[sl["slot"]], sl["degree"], prog, kinds))
    return out


def _m125_replay_slots(SP):
    cs = iter(splitmix_fp(95, 1 << 16).tolist())

    def coef(cls):
        return "one" if cls == "one" else (next(cs) % (1 << 40), 0) if cls == "kbase" else (next(cs), next(cs))

    out = []
    for sl in _m125_slots():
        kinds = ["eq"] + ["base" if f == "base" else "ext" for f in sl["table_fields"][1:]]
        out.append((sl["name"], sl["main_rounds"], sl["declared_degree"], _program_from_structure(SP, sl, coef), kinds))
    return out


def slot_replay(dev, backend, st, rows, n, slots, shape_note) -> dict:
    """All 23 slot sumchecks of one block, replayed on the device: per slot the tables are built ON THE DEVICE from the
    resident rows of a commitment (an eq cube for an eq table, committed planes for the rest: base-valued where the reference
    records a base table, partially evaluated at one fixed coordinate where it records an extension table), then the masked
    sumcheck runs with the device Fiat-Shamir step.  Points and plane positions are seeded; the graphs, table counts and degrees
    are the reference's.  This is device WORK of the stated shape, not a proof: the protocol layer that would drive it is the
    reference's Rust crate."""
    ctx = dev.ctx
    words_avail = rows * n
    per_slot, total_tables_ms, total_rounds_ms, total_bytes = {}, 0.0, 0.0, 0
    cs = iter(splitmix_fp(96, 1 << 16).tolist())
    for name, nv, deg, prog, kinds in slots:
        k = len(kinds)
        point = np.array([next(cs) for _ in range(2 * nv)], dtype=np.uint64).reshape(nv, 2)
        mask = np.array([next(cs) for _ in range(2 * ((nv + 1) * deg + 2))], dtype=np.uint64).reshape(-1, 2)
        ctx.timing_read(reset=True)
        tabs = backend.B200Tables(ctx, k, nv)
        for t in range(k):
            if kinds[t] == "eq":
                tabs.plan_eq(t, point, 0)
                continue
            if kinds[t] == "base":
                coords, span = [("rho", v) for v in range(nv)], 1 << nv
            else:
                coords, span = [("fixed", (next(cs), next(cs)))] + [("rho", v) for v in range(nv)], 2 << nv
            off = (next(cs) % max(1, words_avail - span)) if span < words_avail else 0
            tabs.plan_plane(t, st, coords, [(int(off), (1, 0))])
        ev = backend.B200Rounds(ctx, prog, tabs, deg)
        ev.batched(nv, bytes(32), 0, None, mask=mask, mask_vars=nv + 1, mask_c=(3, 5), recover_one=True, claim=(0, 0))
        ev.free()
        tm = ctx.timing_read(reset=True)
        per_slot[name] = {"rounds": nv, "tables": k, "degree": deg, "tables_ms": round(tm["tables"][0], 3), "sumcheck_ms": round(tm["rounds"][0], 3)}
        total_tables_ms += tm["tables"][0]
        total_rounds_ms += tm["rounds"][0]
        total_bytes += k * (16 << nv)
    return {"slots": len(slots), "tables_ms": total_tables_ms, "sumchecks_ms": total_rounds_ms, "table_bytes": total_bytes, "per_slot": per_slot,
            "shape": shape_note}


def cpu_extras(o, backend, np_data) -> dict:
    """The same operations as `device_extras` on the host cores through the CPU restatement (OpenMP where the reference
    uses rayon), each on the sample named in its key's note; milliseconds scaled to the full operation."""
    w = WORK
    n, rows = 1 << w["log_cols"], w["rows"]
    out, notes = {}, {}

    def timed(f):
        t0 = time.perf_counter()
        f()
        return (time.perf_counter() - t0) * 1e3

    rhos = splitmix_fp(77, 4 * rows * 2).reshape(4, rows, 2)
    out["open_A_fold_38rho_ms"] = timed(lambda: o.fold_rows(np_data, rows, n, n, 1, rhos)) * 38 / 4
    notes["open_A_fold_38rho_ms"] = "4 of 38 vectors over the message columns, scaled"
    srho = structured_rhos(splitmix_fp(77, 38 * rows * 2).reshape(38, rows, 2))
    out["open_A_fold_37_plane_vectors_1_dense_ms"] = timed(lambda: o.fold_rows(np_data, rows, n, n, 1, srho))
    notes["open_A_fold_37_plane_vectors_1_dense_ms"] = "message columns only; the restatement skips zero weights as the reference does"
    nv = 21
    tables = splitmix_fp(79, 3 * (1 << nv) * 2).reshape(3, 1 << nv, 2)
    alpha = splitmix_fp(80, 2).reshape(1, 2)
    mask = splitmix_fp(81, ((nv + 1) * 3 + 2) * 2).reshape(-1, 2)
    out["sumcheck_logup_q_2^21_deg3_21rounds_ms"] = timed(lambda: o.sc_prove(o.POLY_LOGUP_Q, tables, 3, o.Transcript(b"bench"), coefs=alpha, mask=mask,
                                                                             mask_c=(3, 5), mask_vars=nv + 1, recover_one=True, claim=(0, 0)))
    nq = 1 << 21
    qidx = (splitmix_fp(82, nq) % np.uint64(1 << 16)).astype(np.int32)
    qout = (splitmix_fp(83, nq) % np.uint64(1 << 15)).astype(np.int32)
    out["logup_helpers_2^21_ms"] = timed(lambda: o.logup_helpers(qidx, qout, (11, 12), (13, 14), (15, 16)))
    wm = (splitmix_fp(84, 4096 * 14336) % np.uint64(256)).astype(np.uint8).view(np.int8).reshape(4096, 14336)
    cw = splitmix_fp(85, 14336 * 2).reshape(14336, 2)
    out["fold_cols_i8_4096x14336_ms"] = timed(lambda: o.fold_cols_i8(wm, cw))
    rw = splitmix_fp(89, 4096 * 2).reshape(4096, 2)
    out["fold_rows_i8_4096x14336_ms"] = timed(lambda: o.fold_rows_i8(wm, rw))
    npair = 1 << 22
    la = (splitmix_fp(92, npair) % np.uint64(256)).astype(np.int64)
    lb = (splitmix_fp(93, npair) % np.uint64(256)).astype(np.int64)

    def lookup():
        ta, tb = o.lookup_inverse_table((21, 22), (23, 24), 256), o.lookup_inverse_table((21, 22), (25, 26), 256)
        o.lookup_helpers(la, ta, (23, 24), (21, 22), b=lb, tab_b=tb, g_b=(25, 26))

    rngw = np.random.default_rng(5)
    xw, ww = rngw.integers(-32768, 32768, 128 * 4096, dtype=np.int64), rngw.integers(-128, 128, 4096 * 1024, dtype=np.int8)
    out["witness_products_8B_block_T128_ms"] = timed(lambda: o.witness_product(128, xw, 4096, ww, 4096, 1024, 1024, 128 * 1024, False)) * (218103808 / 4194304)
    notes["witness_products_8B_block_T128_ms"] = "the k projection (128 x 4096 x 1024) on all cores, scaled by weight count to the block's seven products"
    specs = [(21, 3)] * 12 + [(19, 5)] * 8 + [(14, 2)] * 4
    tg = o.HashTag.for_profile(w["profile"])
    box = {}
    out["mask_M_24masks_commit_and_tree_wall_ms"] = timed(lambda: box.setdefault("mc", o.mask_commit(specs, o.ZkRng(3, b"bench-mask"), tg)))
    fr = o.ZkRng(4, b"bench-mask-f")
    fs = [((1, 2), [(s_, fr.fp2_vec(specs[s_][0] * specs[s_][1] + 2))]) for s_ in range(len(specs))]
    out["mask_M_24masks_open_wall_ms"] = timed(lambda: o.mask_open(box["mc"], fs, o.Transcript(b"bench-mask")))
    notes["mask_M_24masks_open_wall_ms"] = "numpy restatement (transforms and hashing in C, one thread; includes the functionals' weight combination)"
    out["lookup_helpers_u8_pairs_2^25_ms"] = timed(lookup) * 8
    notes["lookup_helpers_u8_pairs_2^25_ms"] = "2^22 of 2^25 pairs, scaled"
    g = o.ZkRng(1, b"bench")
    out["draw_pads_and_salts_of_A_ms"] = timed(lambda: (g.fp_vec(rows * w["q"]), g.salts(n * w["inv_rate"])))
    notes["draw_pads_and_salts_of_A_ms"] = "one thread, as the reference draws them (pcs.rs:788-792)"
    point = splitmix_fp(90, 21 * 2).reshape(21, 2)
    coords = [("fixed", (int(a), int(b))) for a, b in splitmix_fp(91, 6).reshape(3, 2)] + [("rho", k) for k in range(19)]
    out["tables_eq_2^21_plus_plane_2^19_x8_ms"] = timed(lambda: (o.eq_cube(point, 21, 0), o.priv_table(coords, [(0, (1, 0))], np_data, 19)))
    notes["tables_eq_2^21_plus_plane_2^19_x8_ms"] = "walked host builder, one thread"
    prog, deg, base = slot14_program(backend.SlotProgram)
    nv = 19
    tables = slot14_tables(prog, base, nv)
    mask = splitmix_fp(88, ((nv + 1) * deg + 2) * 2).reshape(-1, 2)
    o.ir_set(prog.words(), prog.n_nodes, prog.n_terms)
    out["sumcheck_slot_program_60tables_71nodes_deg5_2^19_ms"] = timed(lambda: o.sc_prove(o.POLY_IR, tables, deg, o.Transcript(b"bench"), coefs=prog.coef_array(),
                                                                                          mask=mask, mask_c=(3, 5), mask_vars=nv + 1, recover_one=True, claim=(0, 0)))
    out["notes"] = notes
    return out


def cpu_verify(o, dev, np_data, np_pads, np_pows, col_key) -> float:
    """The same verifier work on the host through the restatement: 78 row encodings, then hash, path and 39 combinations per column."""
    w = WORK
    n, nn = 1 << w["log_cols"], (1 << w["log_cols"]) * w["inv_rate"]
    rhos38 = splitmix_fp(77, 38 * w["rows"] * 2).reshape(38, w["rows"], 2)
    cols, idx, salts, paths, root, ck, lk, nk, rhos, vecs = verifier_inputs(dev, np_data, np_pads, np_pows, col_key, rhos38)["args"]
    tag = o.HashTag(transcript=None, column=ck, leaf=lk, node=nk)
    t0 = time.perf_counter()
    enc = [(o.encode_row_zk(v[:n, 0], v[n:, 0], np_pows, w["log_cols"] + 1), o.encode_row_zk(v[:n, 1], v[n:, 1], np_pows, w["log_cols"] + 1)) for v in vecs]
    verdicts = o.check_columns_host(list(cols), idx, [bytes(x) for x in salts], [[bytes(x) for x in p] for p in paths], root, tag, rhos, enc)
    ms = (time.perf_counter() - t0) * 1e3
    assert verdicts == [0] * len(idx)
    return ms


def extras_rooflines(extras: dict, peak_gbs: float) -> dict:
    """Algorithmic bytes (and field multiply-adds where arithmetic is the bound) of every timed operation of `device_extras`,
    with the achieved rate as a fraction of the measured HBM copy peak.  Bytes are what the operation must read and write once."""
    w = WORK
    n, nn, q, rows = 1 << w["log_cols"], (1 << w["log_cols"]) * w["inv_rate"], w["q"], w["rows"]
    a_bytes = 8 * rows * (n + q)
    spec = {
        "open_A_fold_38rho_ms": (a_bytes + 38 * (n + q) * 16, {"field_multiply_adds": 38 * rows * (n + q) * 2, "bound": "arithmetic (every vector dense: the worst case)"}),
        "open_A_fold_37_plane_vectors_1_dense_ms": (a_bytes + 38 * (n + q) * 16, {"bound": "hbm (the dense proximity vector reads every row once)"}),
        "open_H_fold_9_plane_vectors_1_dense_ms": (a_bytes + 10 * (n + q) * 16, {"bound": "hbm"}),
        "open_A_gather_280cols_ms": (280 * rows * 32, {"bound": "latency (one 32-byte sector per gathered word)"}),
        "sumcheck_logup_q_2^21_deg3_21rounds_ms": (3 * 16 * 3 * (1 << 21), {"bound": "hbm in the long rounds (each round reads its tables, each fold reads and writes them), then launch latency"}),
        "logup_helpers_2^21_ms": ((4 + 4 + 16) << 21, {"bound": "integer (one Fp2 inversion per 8 queries)"}),
        "fold_cols_i8_4096x14336_ms": (4096 * 14336, {"field_multiply_adds": 4096 * 14336 * 2, "bound": "arithmetic (two wide multiply-adds per matrix byte)"}),
        "fold_rows_i8_4096x14336_ms": (4096 * 14336, {"field_multiply_adds": 4096 * 14336 * 2, "bound": "arithmetic"}),
        "draw_pads_and_salts_of_A_ms": (8 * rows * q + 32 * nn, {"bound": "integer (one BLAKE3 compression per 64 bytes)"}),
        "lookup_helpers_u8_pairs_2^25_ms": (32 << 25, {"bound": "hbm"}),
        "tables_eq_2^21_plus_plane_2^19_x8_ms": ((16 << 21) + (16 << 19) + (8 * 8 << 19), {"bound": "hbm"}),
        "sumcheck_slot_program_60tables_71nodes_deg5_2^19_ms": (3 * 16 * 60 * (1 << 19), {"bound": "integer issue (219 products of extension-field values per pair and point)"}),
        "witness_products_8B_block_T128_ms": (218103808 + 7 * 0, {"int8_multiply_adds": 128 * 218103808, "bound": "weights streamed once; launch structure"}),
    }
    out = {}
    for key, (nbytes, more) in spec.items():
        if key in extras and extras[key]:
            gbs = nbytes / (extras[key] * 1e-3) / 1e9
            out[key] = {"ms": extras[key], "algorithmic_bytes": nbytes, "achieved_GBps": gbs, "frac_of_measured_hbm": gbs / peak_gbs, **more}
    return out


def reference_cuda_extras(dev, backend, d_data, d_pads, d_pows, col_key) -> dict:
    """The reference's OWN CUDA kernels (hashline/src/gpu/kernels.cu compiled unchanged for sm_100a, launched as
    hashline/src/gpu/cuda.rs launches them) on this GPU, beside this repository's kernels on the same inputs: device
    milliseconds, CUDA events.  None when the compiled module is absent."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_cuda

    if not ref_cuda.available():
        return None
    w = WORK
    log_cols, ir, q, rows = w["log_cols"], w["inv_rate"], w["q"], w["rows"]
    n, nn = 1 << log_cols, (1 << log_cols) * ir
    ref = ref_cuda.RefCuda(max_log=log_cols + 1)
    ctx = dev.ctx
    cs = torch.cuda.current_stream()

    def timed(f, reps=3):
        f()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(cs)
        for _ in range(reps):
            f()
        b.record(cs)
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    out, mine = {}, {}
    box = {}
    out["encode"] = timed(lambda: box.__setitem__("enc", ref.encode_zk(d_data, d_pads, d_pows, rows, log_cols, log_cols + 1, q)))
    enc = box["enc"]
    out["column_hash"] = timed(lambda: ref.hash_cols(enc, rows, nn, col_key))
    # the reference folds at most 4 vectors per launch over the data columns (cuda.rs:3437-3460): 38 vectors = 10 launches
    rhos = torch.from_numpy(splitmix_fp(77, 4 * rows * 2).view(np.int64)).cuda()
    out["open_A_fold_38rho"] = timed(lambda: [ref.fold_rows(d_data, rhos, rows, n, 4) for _ in range(10)])
    del enc, box
    nv = 21
    tabs = torch.from_numpy(splitmix_fp(79, 3 * (1 << nv) * 2).view(np.int64)).cuda()

    def all_folds():
        half = 1 << (nv - 1)
        while half >= 1:
            ref.sc_fold(tabs, 3, half, 1 << nv, (3, 5))
            half //= 2

    out["sumcheck_folds_3tables_2^21_all_rounds"] = timed(all_folds)
    point = splitmix_fp(90, 21 * 2).reshape(21, 2)
    out["eq_table_2^21"] = timed(lambda: ref.eq_table(point))
    nq = 1 << 21
    a_dev = torch.from_numpy(np.concatenate([splitmix_fp(82, nq) % np.uint64(1 << 16), splitmix_fp(83, nq) % np.uint64(1 << 15),
                                             splitmix_fp(84, nq) % np.uint64(256)]).view(np.int64)).cuda()
    h_dev = torch.empty(2 * nq, dtype=torch.int64, device="cuda")
    out["helper_column_2^21"] = timed(lambda: ref.helper(a_dev, 0, nq, 2 * nq, nq, (11, 12), (13, 14), (15, 16), (17, 18), h_dev, 0, nq))
    del tabs, a_dev, h_dev
    # this repository's kernels on the same operations (library timing classes: kernels only)
    ctx.timing_enable(True)
    tables = splitmix_fp(79, 3 * (1 << nv) * 2).reshape(3, 1 << nv, 2)
    ev = backend.B200Rounds(ctx, backend.POLY_LOGUP_Q, tables, 3, splitmix_fp(80, 2).reshape(1, 2))
    ctx.timing_read(reset=True)
    for _ in range(nv):
        ev.fold((3, 5))
    mine["sumcheck_folds_3tables_2^21_all_rounds"] = ctx.timing_read(reset=True)["rounds"][0]
    ev.free()
    for rep in range(3):
        if rep == 1:
            ctx.timing_read(reset=True)
        t21 = backend.B200Tables(ctx, 1, 21)
        t21.plan_eq(0, point, 0)
        t21.flush()
        t21.free()
    mine["eq_table_2^21"] = ctx.timing_read(reset=True)["tables"][0] / 2
    ctx.timing_enable(False)
    return {"ms": out, "this_repository_ms": mine,
            "note": "reference kernels: k_ntt_p1/k_ntt_p2_f/k_zk_pad_scale (encode), k_hash_cols_keyed, k_fold_rows x10, k_sc_fold x21, k_eq_table + k_eq_join, "
                    "k_helper; this repository's figures for encode, column hash, the opening fold and the helper column are kernel_ms_per_step and "
                    "other_kernels_device_ms of the same line"}


def block_device_trace(line: dict, extras: dict, commit_h_ms: float) -> dict:
    """A MODEL of one block's device time at the Llama-3-8B block shape, summed from measured device times of this run, with
    host work = 0 and no overlap between steps: the per-block call list of a W16R2_8B_T128_H24 block core (commit A, LogUp
    helper columns, commit H, commit M, 23 slot sumchecks with their tables, openings of M, A and H, the witness products and
    the public weight folds).  It is not a measurement of proved tokens per second: the protocol layer that drives these calls
    is the reference's Rust crate."""
    rep = extras["slot_replay_8B_T128"]
    steps = {
        "commit_A_2504x2^14": line["ms_per_step"],
        "commit_H_2606x2^14": commit_h_ms,
        "commit_M_24_masks_and_tree": extras["mask_M_24masks_commit_and_tree_wall_ms"],
        "helper_columns_32M_looked_words": extras["lookup_helpers_u8_pairs_2^25_ms"] * 0.5,
        "helper_columns_exp_and_activation_2.6M_inversions": extras["logup_helpers_2^21_ms"] * 2.6 / 2.1,
        "slot_tables_1.44GB": rep["tables_ms"],
        "slot_sumchecks_23": rep["sumchecks_ms"],
        "open_M": extras["mask_M_24masks_open_wall_ms"],
        "open_A_38_vectors_280_columns": extras["open_A_fold_37_plane_vectors_1_dense_ms"] + extras["open_A_gather_280cols_ms"],
        "open_H_10_vectors_280_columns": extras["open_H_fold_9_plane_vectors_1_dense_ms"] * 2606 / 2504 + extras["open_A_gather_280cols_ms"],
        "witness_products_7": extras["witness_products_8B_block_T128_ms"],
        "public_weight_folds_218MB_int8": extras["fold_cols_i8_4096x14336_ms"] * 218103808 / (4096 * 14336),
    }
    block_ms = sum(steps.values())
    blocks, tokens = 32, 128
    request_ms = blocks * block_ms
    return {"model": True, "label": "MODEL, not a measurement: sum of this run's measured device times, host work = 0, no overlap, no boundary commitments or join",
            "shape": "W16R2_8B_T128_H24: one block of Llama-3-8B shapes, 128 tokens", "steps_ms": {k: round(v, 4) for k, v in steps.items()},
            "block_device_ms": block_ms, "blocks_per_request": blocks, "request_device_ms": request_ms,
            "modelled_device_only_tokens_per_s": tokens / (request_ms * 1e-3),
            "reference_published": "22.9 - 34.2 proved tokens/s on an Apple M3 Ultra (whole prover, host work included)"}


D55_BLOCKS = 8
# S1 of the bench's D55 run (below) proved by ONE process; every world size must join to the same state (run_fork.rs:1819-1827)
D55_EXPECTED_S1 = "5af4ea9224dd48e403b182d2267a79b80245dd0e8ce75e10d7a9a64ccfc3e848"


def d55_leg(dev, backend, rank: int, world: int, col_key, leaf_key, node_key) -> dict:
    """A D55 commit-fork-join run with its work on the device: rank 0 commits the boundary planes and broadcasts their roots;
    D55_BLOCKS blocks, block k proved by rank k mod world (a
    hiding commitment with its tree, an opening and a masked sumcheck with the device Fiat-Shamir step per fork:
    d55.device_fork), the fixed-size join records all-gathered over NCCL, the join replayed on every rank.  Returns S1 and the
    wall time; S1 does not depend on the world size."""
    import torch
    import torch.distributed as dist
    from intelligenceregulation_b200 import d55

    lc, ir, rows, q, nv = 12, 2, 296, 64, 14
    nn = ir << lc
    pows = coset_powers(nn)
    header = d55.RunHeader(WORK["profile"].encode(), col_key, D55_BLOCKS, (128, 4096, 14336, 32, 8, 128), b"\x01" * 64, b"\x02" * 32, b"bench", b"\x03" * 16,
                           b"\x04" * 32)
    digs = [bytes([64 + k]) * 32 for k in range(D55_BLOCKS)]
    brows = 32 + 2 * 2 + 2  # a boundary plane: 32 data rows, a reserved row pair per claim site, a proximity pair (boundary.rs:184-188)

    def commit_plane(b):  # rank 0 only: a few rows, so the encoder's one-CTA-per-(row, residue) form
        salts = (splitmix_fp(0xD5C00 + b, nn * 4).view(np.uint8)).reshape(nn, 32)
        st, _, levels = dev.try_commit_zk_tree(lc, ir, witness_words(0xD5A00 + b, brows, 1 << lc), splitmix_fp(0xD5B00 + b, brows * q), pows, lc + 1, col_key, salts,
                                               leaf_key, node_key, want_leaves=False)
        st.free()
        return bytes(levels[-1])

    def bcast(buf):
        nbytes = 1 + 32 * (D55_BLOCKS - 1)
        t = torch.frombuffer(bytearray(buf), dtype=torch.uint8).cuda() if rank == 0 else torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        dist.broadcast(t, src=0)
        return t.cpu().numpy().tobytes()

    def block(k):
        return dict(log_cols=lc, inv_rate=ir, data=witness_words(0xD5500 + k, rows, 1 << lc), pads=splitmix_fp(0xD5600 + k, rows * q),
                    salts=(splitmix_fp(0xD5700 + k, nn * 4).view(np.uint8)).reshape(nn, 32), pows=pows, keys=(col_key, leaf_key, node_key),
                    tables=splitmix_fp(0xD5800 + k, 4 * (1 << nv) * 2).reshape(4, 1 << nv, 2), mask=splitmix_fp(0xD5900 + k, ((nv + 1) * 3 + 2) * 2).reshape(-1, 2))

    def gather(buf):
        mine = torch.frombuffer(bytearray(buf), dtype=torch.uint8).cuda()
        out = torch.empty(world * mine.numel(), dtype=torch.uint8, device="cuda")
        dist.all_gather_into_tensor(out, mine)
        host = out.cpu().numpy().tobytes()
        return [host[i * len(buf):(i + 1) * len(buf)] for i in range(world)]

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    roots = d55.commit_boundaries(commit_plane, D55_BLOCKS, rank, world, bcast if world > 1 else None)
    s1 = d55.run_forks(header, roots, [brows] * (D55_BLOCKS - 1), [lc] * (D55_BLOCKS - 1), digs,
                       lambda k, tr: d55.device_fork(dev, backend, k, tr, block(k)), rank, world, gather if world > 1 else None)
    wall = time.perf_counter() - t0
    out = {"blocks": D55_BLOCKS, "s1": s1.state.hex(), "counter": s1.counter, "wall_ms": wall * 1e3,
           "fork": f"commit {rows} x 2^{lc} -> 2^{lc + 1} with tree, opening (1 combination, 8 columns), masked zero-check sumcheck of 2^{nv} points",
           "boundaries": f"{D55_BLOCKS - 1} planes of {brows} x 2^{lc} committed on rank 0, their roots in one broadcast",
           "exchange": "one broadcast of the boundary roots, one all-gather of fixed-size join records, over NCCL" if world > 1 else "none (one process)"}
    if D55_EXPECTED_S1 is not None:
        assert out["s1"] == D55_EXPECTED_S1, "the D55 join state differs from the one-process value"
        out["s1_equals_one_process_value"] = True
    return out


def run_b200(args, rank: int, local_rank: int, world: int) -> None:
    import torch
    import torch.distributed as dist
    from intelligenceregulation_b200 import backend

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this backend has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    w = WORK
    log_cols, ir, q, rows = w["log_cols"], w["inv_rate"], w["q"], w["rows"]
    n, nn = 1 << log_cols, (1 << log_cols) * ir
    # the bench profile's hash-tag keys (hashtag.rs:47-53,92-100): derive_key is the caller's host logic
    import blake3 as b3

    prof = w["profile"].encode()
    col_key = b3.blake3(prof, derive_key_context="hashline-zk-mr1 2026-09-20 pcs column digest").digest()
    leaf_key = b3.blake3(prof, derive_key_context="hashline-zk-mr1 2026-09-20 pcs salted merkle leaf").digest()
    node_key = b3.blake3(prof, derive_key_context="hashline-zk-mr1 2026-09-20 pcs merkle inner node").digest()

    # this rank's block (D55: block k -> rank k mod world); seeded synthetic witness words uniform in [0, p)
    block = rank
    blk_data, blk_pads, blk_salts = block_inputs(block)
    h_data = torch.from_numpy(blk_data.view(np.int64)).pin_memory()
    h_pads = torch.from_numpy(blk_pads.view(np.int64)).pin_memory()
    h_pows = torch.from_numpy(coset_powers(nn).view(np.int64)).pin_memory()
    h_salts = torch.from_numpy(blk_salts).pin_memory()
    # the same rows as the prover's uploader sends them: every row at the narrowest width that holds it, page-locked
    packed_np, row_width = backend.pack_rows(blk_data, rows)
    h_packed = torch.from_numpy(packed_np).pin_memory()
    np_packed = h_packed.numpy()
    del packed_np, blk_data, blk_pads

    dev = backend.B200Backend(device=local_rank)
    stream = torch.cuda.Stream()  # the library, torch's copies and the timing events all use this one stream
    torch.cuda.set_stream(stream)
    dev.ctx.set_stream(stream.cuda_stream)
    d_data, d_pads, d_pows, d_salts = (t.cuda(non_blocking=True) for t in (h_data, h_pads, h_pows, h_salts))
    d_levels = torch.empty((2 * nn - 1) * 32, dtype=torch.uint8, device="cuda")
    roots = torch.empty(world * 32, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()

    def step_resident():
        st = dev.commit_zk_dev(log_cols, ir, d_data.data_ptr(), rows, d_pads.data_ptr(), q, d_pows.data_ptr(), col_key)
        st.merkle_dev(d_salts.data_ptr(), leaf_key, node_key, d_levels.data_ptr())
        st.free()
        if world > 1:
            dist.all_gather_into_tensor(roots, d_levels[-32:])

    np_data, np_pads, np_pows, np_salts = (t.numpy().view(np.uint64) if t.dtype == torch.int64 else t.numpy() for t in (h_data, h_pads, h_pows, h_salts))

    e2e_parts = [0.0, 0.0, 0.0]  # this rank's wall time in the commitment call, the tree call, the exchange of roots

    # the caller's result buffers, page-locked like its inputs
    np_levels = torch.empty((2 * nn - 1) * 32, dtype=torch.uint8).pin_memory().numpy().reshape(2 * nn - 1, 32)

    def step_e2e(wide: bool = False):
        t0 = time.perf_counter()
        if wide:  # the 64-bit upload (hl_b200_commit_zk_tree), for the comparison line only
            st, leaves, levels = dev.try_commit_zk_tree(log_cols, ir, np_data, np_pads, np_pows, log_cols + 1, col_key, np_salts.reshape(nn, 32), leaf_key,
                                                        node_key, levels_out=np_levels, want_leaves=False)
        else:
            st, leaves, levels = dev.try_commit_zk_packed(log_cols, ir, np_packed, row_width, np_pads, np_pows, log_cols + 1, col_key, np_salts.reshape(nn, 32),
                                                          leaf_key, node_key, levels_out=np_levels, want_leaves=False)
        t1 = time.perf_counter()
        st.free()
        t2 = time.perf_counter()
        if world > 1:
            dist.all_gather_into_tensor(roots, torch.from_numpy(levels[-1].copy()).cuda())
            stream.synchronize()
        e2e_parts[0] += t1 - t0
        e2e_parts[1] += t2 - t1
        e2e_parts[2] += time.perf_counter() - t2
        return leaves, levels

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.profile_extras:
        if rank == 0:
            print(json.dumps({"profile_run": True, "only": args.only, "other_kernels_device_ms": device_extras(dev, backend, np_data, np_pads, np_pows, col_key, args.only)}))
        dev.ctx.close()
        return

    # ---- resident-input leg ----
    # one sampling process for all the job's GPUs, on rank 0: every query takes the driver's lock, and one process per
    # rank stalled the other ranks' copies and allocations
    sampler = ClockSampler(range(world) if rank == 0 else [])
    sampler.start()
    for _ in range(args.warmup):
        step_resident()
    barrier()
    dev.ctx.timing_read(reset=True)
    dev.ctx.timing_enable(True)
    launches0 = dev.ctx.stats()["kernel_launches"]
    sampler.rows.clear()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    e0.record(stream)
    marks[0].record(stream)
    for k in range(args.steps):
        step_resident()
        marks[k + 1].record(stream)
    e1.record(stream)
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    per_step = sorted(marks[k].elapsed_time(marks[k + 1]) for k in range(args.steps))
    tim = dev.ctx.timing_read(reset=True)
    dev.ctx.timing_enable(False)
    launches = dev.ctx.stats()["kernel_launches"] - launches0
    root_resident = bytes(d_levels[-32:].cpu().numpy())

    if args.profile:
        sampler.stop()
        if rank == 0:
            print(json.dumps({"profile_run": True, "ms_per_step": ms / args.steps, "kernel_ms": {k: v[0] / max(1, v[1]) for k, v in tim.items()}, "gpu_launches": launches}))
        dev.ctx.close()
        return

    # ---- end-to-end leg: host pointers in, leaves + tree out ----
    for _ in range(max(1, args.warmup // 2)):
        step_e2e()
    barrier()
    s0 = dev.ctx.stats()
    t0 = time.perf_counter()
    e2e_parts[:] = [0.0, 0.0, 0.0]
    for _ in range(args.steps):
        leaves, levels = step_e2e()
    barrier()
    e2e_own = time.perf_counter() - t0
    parts_timed = list(e2e_parts)  # this leg's parts only: the 64-bit comparison below runs through the same function
    e2e_s = max_over_ranks(e2e_own)
    clocks = sampler.stop()
    s1 = dev.ctx.stats()
    assert bytes(levels[-1]) == root_resident, "the two legs disagree on the root"
    # the same call with the rows as 64-bit words (what the end-to-end leg cost before the narrow upload), a few steps
    wide_steps = min(args.steps, 8)
    step_e2e(wide=True)
    barrier()
    tw0 = time.perf_counter()
    for _ in range(wide_steps):
        _, levels_w = step_e2e(wide=True)
    barrier()
    e2e_wide_ms = max_over_ranks((time.perf_counter() - tw0) * 1e3 / wide_steps)
    assert bytes(levels_w[-1]) == root_resident, "the wide upload disagrees on the root"

    # what the upload alone costs on this box: the same pinned buffers, one copy each, nothing else on the device
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    d_packed = torch.empty_like(h_packed, device="cuda")
    d_packed.copy_(h_packed, non_blocking=True)
    barrier()  # every rank copies at the same time, as in the leg above: the ranks share the host's upload path
    c0.record(stream)
    for _ in range(5):
        d_packed.copy_(h_packed, non_blocking=True)
        d_pads.copy_(h_pads, non_blocking=True)
        d_salts.copy_(h_salts, non_blocking=True)
    c1.record(stream)
    torch.cuda.synchronize()
    h2d_only_ms = c0.elapsed_time(c1) / 5
    del d_packed
    per_rank = None
    if world > 1:  # every rank's own wall time and upload time: the ranks share the host's memory and PCIe root complexes
        t = torch.tensor([e2e_own * 1e3 / args.steps, h2d_only_ms] + [x * 1e3 / args.steps for x in parts_timed], dtype=torch.float64, device="cuda")
        allt = torch.empty(5 * world, dtype=torch.float64, device="cuda")
        dist.all_gather_into_tensor(allt, t)
        per_rank = [[round(x, 3) for x in row] for row in allt.view(world, 5).tolist()]

    enc_bytes = rows * nn * 8
    value = world * enc_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e_v = world * enc_bytes * args.steps / e2e_s / 1e9
    enc_ms = tim["encode"][0] / max(1, tim["encode"][1])
    hash_ms = tim["hash"][0] / max(1, tim["hash"][1])
    mer_ms = tim["merkle"][0] / max(1, tim["merkle"][1])
    alg_bytes = 8 * rows * (n + q) + 8 * rows * nn
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = alg_bytes / (enc_ms * 1e-3) / 1e9

    cpu = None
    if world == 1 and rank == 0:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import hl_oracle as o

        if "LOCAL_RANK" in os.environ:
            o.set_threads(len(os.sched_getaffinity(0)))
        # the SAME matrix, pads and salts on the host cores: the CPU root must be the GPU root; repeated for about ten seconds
        sec, cpu_root = cpu_commit(o, np_data, np_pads, np_salts)
        assert cpu_root == root_resident, "the CPU restatement and the device disagree on the root of the bench's own matrix"
        reps, spent = 1, sec
        while spent < 10.0 and reps < 30:
            s2, _ = cpu_commit(o, np_data, np_pads, np_salts)
            sec, spent, reps = min(sec, s2), spent + s2, reps + 1
        cpu = {"value": rows * nn * 8 / sec / 1e9, "unit": "GB/s", "cores": o.num_threads(), "kind": "port", "root_equals_gpu_root": True,
               "sample": f"best of {reps} commitments ({spent:.1f} s): " + CPU_NOTE.format(rows=rows)}

    # integer ceiling: the same butterfly arithmetic on registers only; radix-2 butterflies of one encoder launch:
    # rows * (1 + R) * (n/2) log2 n (one inverse and R forward size-n transforms per row)
    compress_peak = dev.ctx.compress_peak(400)
    # compressions of one column hash: per column ceil(rows * 8 / 64) blocks and (chunks - 1) parent nodes
    hash_compressions = nn * ((rows * 8 + 63) // 64 + (rows + 127) // 128 - 1)
    bfly_peak = dev.ctx.butterfly_peak(400)
    bfly_per_launch = rows * (1 + ir) * (n // 2) * log_cols
    d55_out = d55_leg(dev, backend, rank, world, col_key, leaf_key, node_key)
    extras = device_extras(dev, backend, np_data, np_pads, np_pows, col_key) if (world == 1 and rank == 0 and not args.no_extras) else None
    extras_cpu = cpu_extras(o, backend, np_data) if extras is not None else None
    if extras_cpu is not None:
        extras_cpu["verify_280_columns_39_vectors_wall_ms"] = cpu_verify(o, dev, np_data, np_pads, np_pows, col_key)
        extras_cpu["notes"]["verify_280_columns_39_vectors_wall_ms"] = "the restated verifier's column part, one thread (the reference runs the columns on rayon)"
    ref_cuda_ms = reference_cuda_extras(dev, backend, d_data, d_pads, d_pows, col_key) if extras is not None else None

    if rank == 0:
        line = {
            "metric": "ligero_commit_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "ms_per_step_median": per_step[len(per_step) // 2], "ms_per_step_min": per_step[0], "higher_is_better": True, "scaling": "weak", "vs_baseline": value / world / PUBLISHED_GBPS if world == 1 else None,
            "dtype": "u64", "data": "synthetic", "config": workload_config(world),
            "e2e": {"value": e2e_v, "unit": "GB/s", "h2d_bytes_per_step": (s1["bytes_h2d"] - s0["bytes_h2d"]) // args.steps,
                    "d2h_bytes_per_step": (s1["bytes_d2h"] - s0["bytes_d2h"]) // args.steps, "ms_per_step": e2e_s * 1e3 / args.steps,
                    "h2d_only_ms": h2d_only_ms, "call": "hl_b200_commit_zk_packed (rows as 2-byte / 8-byte words, widened on the device)",
                    "wide_u64_upload": {"call": "hl_b200_commit_zk_tree", "ms_per_step": e2e_wide_ms, "h2d_bytes_per_step": 8 * rows * (n + q) + nn * 40,
                                        "value": world * rows * nn * 8 / (e2e_wide_ms * 1e-3) / 1e9}, **({"per_rank_ms": {"columns": ["step", "h2d_only", "commit_and_tree_call", "store_free", "root_exchange"], "rows": per_rank}} if per_rank else {})},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "k_encode_fast<14,1024>", "achieved": achieved, "peak": peak,
                         "peak_source": "MEASURED_PEAKS.json hbm_gbs" if peaks else "fallback 6650 GB/s", "unit": "GB/s", "frac": achieved / peak,
                         "frac_of_nominal_8000_GBps": achieved / 8000.0,
                         "traffic": encode_dram_traffic(), "traffic_source": "profiles/k_encode_fast_8b_A.json (ncu capture of this kernel at this workload)",
                         "algorithmic_bytes_per_launch": alg_bytes, "ms_per_launch": enc_ms,
                         "note": "integer-issue bound kernel (64-bit modular multiplies on the IMAD pipe); HBM fraction reported as the contract asks"},
            "integer_roofline": {"kernel": "k_encode_fast<14,1024>", "unit": "Gbutterfly/s", "achieved": bfly_per_launch / (enc_ms * 1e-3) / 1e9,
                                 "peak": bfly_peak / 1e9, "frac": bfly_per_launch / (enc_ms * 1e-3) / bfly_peak,
                                 "peak_source": "hl_b200_butterfly_peak: the encoder's own butterfly arithmetic, register resident, all SMs, measured in this run"},
            "column_hash_rooflines": {
                "kernel": "k_hash_col_chunks + k_hash_col_merge", "ms_per_launch": hash_ms,
                "hbm": {"achieved": rows * nn * 8 / (hash_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s", "frac": rows * nn * 8 / (hash_ms * 1e-3) / 1e9 / peak,
                        "algorithmic_bytes_per_launch": rows * nn * 8},
                "integer": {"achieved": hash_compressions / (hash_ms * 1e-3) / 1e9, "peak": compress_peak / 1e9, "unit": "Gcompression/s",
                            "frac": hash_compressions / (hash_ms * 1e-3) / compress_peak,
                            "peak_source": "hl_b200_compress_peak: register-resident BLAKE3 compressions, all SMs, measured in this run"}},
            "kernel_ms_per_step": {"encode": enc_ms, "column_hash": hash_ms, "salt_and_tree": mer_ms},
            "cpu_baseline": cpu,
            "other_kernels_device_ms": extras,
            "other_kernels_rooflines": extras_rooflines(extras, peak) if extras else None,
            "other_kernels_cpu_ms": extras_cpu,
            "reference_cuda_ms": ref_cuda_ms,
            "d55": d55_out,
            "root": root_resident.hex(),
        }
        if extras:
            line["block_device_trace_8B_T128"] = block_device_trace(line, extras, extras["commit_H_2606x2^14_to_root_ms"])
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    dev.ctx.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the device times of the opening, sumcheck and LogUp kernels")
    ap.add_argument("--profile", action="store_true", help="resident-input leg only (for a run under a profiler)")
    ap.add_argument("--profile-rows", type=int, default=0, help="with --profile: commit this many rows instead of the workload's (a capture small enough for multi-pass counters)")
    ap.add_argument("--profile-extras", action="store_true", help="opening, sumcheck and LogUp kernels only (for a run under a profiler)")
    ap.add_argument("--only", default="", help="with --profile-extras: comma-separated families to run (open, sumcheck, helpers, i8folds, rng, lookup, slots, "
                                               "slot_program, mask, witness, long_rows, commit_h, verify)")
    args = ap.parse_args()
    if args.profile and args.profile_rows > 0:
        WORK["rows"] = args.profile_rows
    rank, local_rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_b200(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
