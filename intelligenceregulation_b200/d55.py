"""Host logic of the D55 commit-fork-join run over several GPUs.

The reference proves one request's transformer blocks as independent forks of one transcript
(hashline/src/private_block/run_fork.rs:1617-1860): a commit phase absorbs the L - 1 boundary roots into
S0, every block k is proved from ``fork(S0, k)``, and the join absorbs each fork's end state and IO claims
in block order into S1.  There the forks are threads of one process; here a rank is a GPU, block k belongs
to rank ``k mod world``, and the only data that crosses ranks are the small records below:

* before the forks: the L - 1 boundary roots (32 bytes each), broadcast from rank 0;
* after the forks: one fixed-size join record per block (index, 32-byte state, squeeze counter, two claim
  lists), all-gathered; rank 0 (or every rank) replays the join.

The transcript here is the caller's host transcript (transcript.rs:29-167) over the ``blake3`` package; the
absorbed bytes and labels are those of run_fork.rs:907-1045 (`D55_LABELS` :156-166).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import blake3 as _b3

P = 0xFFFFFFFF00000001


class HostTranscript:
    """transcript.rs:29-167 (no masker): 32-byte state, labelled absorbs, counter-mode squeezes."""

    def __init__(self, domain: bytes, key: Optional[bytes] = None):
        self.key = key
        self.state = self._h(b"hashline-v1/" + domain)
        self.counter = 0

    def _h(self, data: bytes) -> bytes:
        return (_b3.blake3(data, key=self.key) if self.key else _b3.blake3(data)).digest()

    def clone(self) -> "HostTranscript":
        t = HostTranscript.__new__(HostTranscript)
        t.key, t.state, t.counter = self.key, self.state, self.counter
        return t

    def absorb(self, label: bytes, data: bytes) -> None:
        self.state = self._h(self.state + struct.pack("<Q", len(label)) + label + struct.pack("<Q", len(data)) + data)

    def absorb_u64(self, label: bytes, v: int) -> None:
        self.absorb(label, struct.pack("<Q", v))

    def squeeze(self) -> bytes:
        out = self._h(self.state + b"squeeze" + struct.pack("<Q", self.counter))
        self.counter += 1
        self.state = out
        return out

    def challenge_fp2(self) -> Tuple[int, int]:
        b = self.squeeze()
        return (int.from_bytes(b[:16], "little") % P, int.from_bytes(b[16:], "little") % P)


@dataclass
class RunHeader:
    """The public header of a fork run (run_fork.rs:907-922)."""
    profile: bytes
    key: Optional[bytes]
    blocks: int                       # L
    shape: Tuple[int, int, int, int, int, int]  # tokens, width, hidden, q_heads, kv_heads, head_dim
    expected_io: bytes
    public_statement: bytes
    parameter_line: bytes
    calibration: bytes
    schedule_digest: bytes

    def transcript(self) -> HostTranscript:
        tr = HostTranscript(self.profile, self.key)
        tr.absorb(b"run-shape", b"".join(struct.pack("<Q", v) for v in (self.blocks, *self.shape)))
        tr.absorb(b"expected-IO", self.expected_io)
        tr.absorb(b"public-statement", self.public_statement)
        tr.absorb(b"parameters", self.parameter_line)
        tr.absorb(b"calibration", self.calibration)
        tr.absorb(b"schedule", self.schedule_digest)
        return tr


def absorb_commit(tr: HostTranscript, blocks: int, roots: Sequence[bytes], rows: Sequence[int], log_cols: Sequence[int]) -> None:
    """run_fork.rs:975-994 with protocol.rs:154-158: the L - 1 boundary roots in order, then `pb-fork-s0`."""
    if len(roots) + 1 != blocks:
        raise ValueError(f"D55: an {blocks}-block run has {blocks - 1} boundary roots, not {len(roots)}")
    for k, root in enumerate(roots):
        tr.absorb_u64(b"pb-fork-commit-root", k)
        tr.absorb(b"B", root)
        tr.absorb_u64(b"rows", rows[k])
        tr.absorb_u64(b"log-cols", log_cols[k])
    tr.absorb_u64(b"pb-fork-s0", blocks)


def fork(s0: HostTranscript, idx: int, block_digest: bytes) -> HostTranscript:
    """run_fork.rs:996-1009: fork(S0, idx)."""
    t = s0.clone()
    t.absorb_u64(b"pb-run-fork", idx)
    t.absorb(b"pb-run-fork-block", block_digest)
    return t


@dataclass
class JoinRecord:
    """What one fork hands to the join (run_fork.rs:1034-1041)."""
    k: int
    state: bytes
    counter: int
    in_claims: bytes    # claim_bytes() of the slot-21 claims
    out_claims: bytes   # claim_bytes() of the slot-22 claims

    def pack(self, claim_cap: int) -> bytes:
        """Fixed-size wire form for an all-gather: lengths first, claim lists zero-padded to claim_cap."""
        if len(self.in_claims) > claim_cap or len(self.out_claims) > claim_cap or len(self.state) != 32:
            raise ValueError("D55: join record does not fit its slot")
        return (struct.pack("<QQQQ", self.k, self.counter, len(self.in_claims), len(self.out_claims)) + self.state
                + self.in_claims.ljust(claim_cap, b"\0") + self.out_claims.ljust(claim_cap, b"\0"))

    @staticmethod
    def size(claim_cap: int) -> int:
        return 32 + 32 + 2 * claim_cap

    @staticmethod
    def unpack(buf: bytes, claim_cap: int) -> "JoinRecord":
        k, counter, li, lo = struct.unpack_from("<QQQQ", buf, 0)
        if li > claim_cap or lo > claim_cap:
            raise ValueError("D55: corrupt join record")
        state = bytes(buf[32:64])
        ic = bytes(buf[64:64 + li])
        oc = bytes(buf[64 + claim_cap:64 + claim_cap + lo])
        return JoinRecord(k, state, counter, ic, oc)


def claim_bytes(claims) -> bytes:
    """run_fork.rs:1011-1030: count, then per claim its value, part count and every part's public words.
    A claim is (value, [(offset, log_size, coef, [point...])]) with Fp2 as (c0, c1)."""
    b = [struct.pack("<Q", len(claims))]
    for value, parts in claims:
        b.append(struct.pack("<QQQ", value[0], value[1], len(parts)))
        for off, log_size, coef, point in parts:
            b.append(struct.pack("<QQQQQ", off, log_size, coef[0], coef[1], len(point)))
            b.extend(struct.pack("<QQ", x[0], x[1]) for x in point)
    return b"".join(b)


def io_claim_list_len(log_plane: int, log_endpoint: int) -> int:
    """run_fork.rs:176-182: the byte length of one IO slot's claim list at a shape."""
    logm = min(log_plane, log_endpoint)
    part = lambda coords: 8 + 8 + 16 + 8 + 16 * coords  # noqa: E731
    return 8 + 16 + 8 + part(log_plane) + 2 * part(logm)


def absorb_join(tr: HostTranscript, rec: JoinRecord) -> None:
    tr.absorb_u64(b"pb-join-fork", rec.k)
    tr.absorb(b"pb-join-state", rec.state + struct.pack("<Q", rec.counter))
    tr.absorb(b"pb-join-in-claims", rec.in_claims)
    tr.absorb(b"pb-join-out-claims", rec.out_claims)


def close_join(tr: HostTranscript, blocks: int) -> None:
    tr.absorb_u64(b"pb-fork-s1", blocks)


def block_owner(k: int, world: int) -> int:
    return k % world


def blocks_of(rank: int, world: int, blocks: int) -> List[int]:
    return [k for k in range(blocks) if block_owner(k, world) == rank]


def join(s0: HostTranscript, records: Sequence[JoinRecord], blocks: int) -> HostTranscript:
    """run_fork.rs:1819-1827: every block exactly once, in block order, then `pb-fork-s1`."""
    by_k = {r.k: r for r in records}
    if len(by_k) != blocks or sorted(by_k) != list(range(blocks)) or len(records) != blocks:
        raise ValueError("D55: the join needs exactly one record per block")
    tr = s0.clone()
    for k in range(blocks):
        absorb_join(tr, by_k[k])
    close_join(tr, blocks)
    return tr


FAILED_K = (1 << 64) - 1  # the `k` word of a record that reports a failed fork instead of a join record


class ForkFailed(RuntimeError):
    """A fork failed on some rank; raised on EVERY rank after the exchange, with the same text."""

    def __init__(self, failures: Sequence[Tuple[int, int, str]]):
        self.failures = list(failures)  # (rank, block, text)
        super().__init__("D55: " + "; ".join(f"block {k} on rank {r}: {t}" for r, k, t in self.failures))


def _failure_record(k: int, text: str, claim_cap: int) -> bytes:
    msg = text.encode("utf-8", "replace")[: 32 + 2 * claim_cap]
    return struct.pack("<QQQQ", FAILED_K, k, len(msg), 0) + msg.ljust(32 + 2 * claim_cap, b"\0")


def commit_boundaries(commit_plane: Callable[[int], bytes], blocks: int, rank: int = 0, world: int = 1,
                      broadcast: Optional[Callable[[Optional[bytes]], bytes]] = None) -> List[bytes]:
    """Phase 1 of a fork run (run_fork.rs:1636-1676): rank 0 commits the L - 1 boundary planes - `commit_plane(b)` returns the
    32-byte root of the plane between blocks b and b + 1 - and the roots reach every rank as ONE broadcast of 32 (L - 1) bytes
    (`broadcast(buffer on rank 0 | None elsewhere) -> buffer`).  Every rank then derives the same S0 from the header and the roots.
    A commitment that fails on rank 0 still takes part in the broadcast, as all-ones roots with a marker, and every rank raises."""
    n = blocks - 1
    buf = None
    if rank == 0:
        try:
            roots = [commit_plane(b) for b in range(n)]
            assert all(len(r) == 32 for r in roots)
            buf = b"\x00" + b"".join(roots)
        except Exception as e:  # noqa: BLE001  (reported to every rank below)
            buf = (b"\x01" + f"{type(e).__name__}: {e}".encode("utf-8", "replace")).ljust(1 + 32 * n, b"\0")[: 1 + 32 * n]
    if world > 1 and broadcast is not None:
        buf = broadcast(buf)
    if buf[0] != 0:
        raise ForkFailed([(0, -1, bytes(buf[1:]).rstrip(b"\0").decode("utf-8", "replace"))])
    return [bytes(buf[1 + 32 * b: 33 + 32 * b]) for b in range(n)]


def run_forks(header: RunHeader, roots: Sequence[bytes], rows: Sequence[int], log_cols: Sequence[int], block_digests: Sequence[bytes],
              prove_fork: Callable[[int, HostTranscript], JoinRecord], rank: int = 0, world: int = 1,
              all_gather: Optional[Callable[[bytes], List[bytes]]] = None, claim_cap: int = 4096) -> HostTranscript:
    """Phase 2 and 3 of a fork run on this rank: prove the blocks this rank owns from fork(S0, k), exchange the
    join records (one fixed-size buffer per rank through `all_gather`), replay the join.  Returns S1.
    A fork that fails does not leave the exchange: its rank still takes part in the gather, with a fixed-size failure
    record in the block's slot (so no healthy rank blocks in a collective a dead peer never joins), stops proving its
    remaining blocks, and every rank raises `ForkFailed` with the same text once the records are in."""
    s0 = header.transcript()
    absorb_commit(s0, header.blocks, roots, rows, log_cols)
    size = JoinRecord.size(claim_cap)
    packed, failed = [], False
    for k in blocks_of(rank, world, header.blocks):
        if failed:
            packed.append(_failure_record(k, "not run: an earlier fork of this rank failed", claim_cap))
            continue
        try:
            packed.append(prove_fork(k, fork(s0, k, block_digests[k])).pack(claim_cap))
        except Exception as e:  # noqa: BLE001  (reported to every rank below)
            failed = True
            packed.append(_failure_record(k, f"{type(e).__name__}: {e}", claim_cap))
    per_rank = -(-header.blocks // world)
    buf = b"".join(packed).ljust(per_rank * size, b"\xff")
    bufs = [buf] if world == 1 or all_gather is None else all_gather(buf)
    records, failures = [], []
    for r, b in enumerate(bufs):
        for i in range(len(blocks_of(r, world, header.blocks))):
            rec = b[i * size:(i + 1) * size]
            k0, k1, mlen, _ = struct.unpack_from("<QQQQ", rec, 0)
            if k0 == FAILED_K:
                failures.append((r, k1, bytes(rec[32:32 + min(mlen, size - 32)]).decode("utf-8", "replace")))
            else:
                records.append(JoinRecord.unpack(rec, claim_cap))
    if failures:
        raise ForkFailed(failures)
    return join(s0, records, header.blocks)


# ----------------------------------------------------------------------------------------------- a fork's device work
def squeeze_index(tr: HostTranscript, bound: int) -> int:
    """one index below the power of two `bound` from one squeeze (transcript.rs:150-167 takes four per squeeze; a fork here
    needs a handful)"""
    return int.from_bytes(tr.squeeze()[:8], "little") & (bound - 1)


def device_fork(dev, backend, k: int, tr: HostTranscript, block: dict) -> JoinRecord:
    """What one block's fork asks of the device, in the order a block proof asks it (protocol.rs:2231-2434 in outline):
    a hiding commitment with its salted tree, the root absorbed; an opening of that commitment at a transcript-drawn
    combination and transcript-drawn columns, absorbed; a masked zero-check sumcheck with the device Fiat-Shamir step
    continuing the fork's transcript.  `block`: log_cols, inv_rate, data, pads, salts, pows, keys (column, leaf, node),
    tables (4 x 2^n x 2), mask.  Everything is a function of (k, transcript, block): whichever rank runs it, the record is
    the same."""
    import numpy as np

    lc, ir = block["log_cols"], block["inv_rate"]
    nn = ir << lc
    rows = block["data"].size >> lc
    ck, lk, nk = block["keys"]
    got = dev.try_commit_zk_tree(lc, ir, block["data"], block["pads"], block["pows"], lc + (ir.bit_length() - 1), ck, block["salts"], lk, nk,
                                 want_leaves=False)
    if got is None:
        raise RuntimeError("D55 fork %d: the device declined the commitment: %s" % (k, dev.ctx.declines[-1][1]))
    store, _, levels = got
    try:
        tr.absorb(b"A", bytes(levels[-1]))
        tr.absorb_u64(b"rows", rows)
        tr.absorb_u64(b"log-cols", lc)
        rho = np.array([tr.challenge_fp2() for _ in range(rows)], dtype=np.uint64).reshape(1, rows, 2)
        fold = store.fold_rows_with_pads(rho)
        tr.absorb(b"pb-open-fold", fold.tobytes())
        idx = np.array([squeeze_index(tr, nn) for _ in range(8)], dtype=np.uint64)
        cols = store.columns(idx)
        tr.absorb(b"pb-open-cols", cols.tobytes())
    finally:
        store.free()
    tables, mask = block["tables"], block["mask"]
    n = int(tables.shape[1]).bit_length() - 1
    tr.absorb_u64(b"pb-slot", k)
    c = tr.challenge_fp2()
    ev = backend.B200Rounds(dev.ctx, backend.POLY_ZC, tables, 3)
    try:
        sums, absorbed, _, state, counter, _ = ev.batched(n, tr.state, tr.counter, tr.key, mask=mask, mask_vars=n + 1, mask_c=c)
        finals = ev.finals()
    finally:
        ev.free()
    # the caller replays the device's rounds through its own transcript (gpu/metal.rs:4156-4171) and must land on the device's state
    for j in range(n):
        tr.absorb(b"sc-round", absorbed[j].tobytes())
        tr.challenge_fp2()
    if tr.state != state or tr.counter != counter:
        raise RuntimeError("D55 fork %d: the device's transcript left the host's" % k)
    tr.absorb(b"pb-term", finals.tobytes())
    value = (int(fold[0, 0, 0]), int(fold[0, 0, 1]))
    point = [(int(a), int(b)) for a, b in rho[0, :min(rows, lc)]]
    ic = claim_bytes([(value, [(0, lc, (1, 0), point)])])
    oc = claim_bytes([((int(finals[0, 0]), int(finals[0, 1])), [(1 << lc, lc, (1, 0), point)])])
    return JoinRecord(k, tr.state, tr.counter, ic, oc)
