"""Oracle for the layer-per-GPU GEMM chain (TEST INFRASTRUCTURE, never on a product path).

Restates, for the CPU:
  * the dependency CSR / scoreboard construction      (reference ctapp/pipeline.py:7-31)
  * the grouped producer tile order                   (reference ctapp/pipeline.py:48-51)
  * the work-queue / scoreboard protocol              (reference csrc/ctapp.cuh:32-69)
  * the chain arithmetic                              (reference tests/test_ctapp.py:33)

Integer artefacts are plain numpy int32 arrays; the arithmetic reference is torch on the CPU with
fp32 accumulation and a bf16 rounding of every inter-stage activation.
"""
from __future__ import annotations

import numpy as np

EMPTY = -1
PAD = 32  # row-panel counters sit one per 128-byte line: 32 int32 apart (ctapp/pipeline.py:29-30)


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def build_deps(M, N1, N2, BM1, BN1, BM2, BN2, rowpanel=True):
    """Dependency CSR over producer tiles (id = m1 * tn1 + n1) and initial scoreboard.

    Producer tile (m1, n1) covers rows [m1*BM1, min((m1+1)*BM1, M)).  Every consumer row panel m2
    whose rows intersect that range depends on it.  In row-panel mode one counter per consumer row
    panel is kept (stored at index m2 * 32); in tile mode one counter per consumer tile
    (id = m2 * tn2 + n2).  Follows reference ctapp/pipeline.py:7-31.
    Returns (dep_offsets[P+1], dep_consumers[nnz], scoreboard_init) as int32 arrays.
    """
    tm1, tn1 = cdiv(M, BM1), cdiv(N1, BN1)
    tm2, tn2 = cdiv(M, BM2), cdiv(N2, BN2)
    offsets = [0]
    consumers = []
    for m1 in range(tm1):
        first_row = m1 * BM1
        last_row = min((m1 + 1) * BM1, M) - 1
        lo, hi = first_row // BM2, last_row // BM2
        for _n1 in range(tn1):
            for m2 in range(lo, hi + 1):
                if rowpanel:
                    consumers.append(m2)
                else:
                    consumers.extend(m2 * tn2 + n2 for n2 in range(tn2))
            offsets.append(len(consumers))
    consumers = np.asarray(consumers, dtype=np.int64)
    n_counters = tm2 if rowpanel else tm2 * tn2
    counts = np.bincount(consumers, minlength=n_counters) if consumers.size else np.zeros(n_counters, np.int64)
    if rowpanel:
        init = np.zeros(tm2 * PAD, dtype=np.int64)
        init[::PAD] = counts
    else:
        init = counts
    return (np.asarray(offsets, dtype=np.int32), consumers.astype(np.int32), init.astype(np.int32))


def producer_order(P, tn1, group_rows=0):
    """Order in which the producer's source queue lists its tile ids (reference ctapp/pipeline.py:48-51).

    group_rows == 0: ascending ids.  Otherwise tile rows are taken in groups of ``group_rows``; inside
    a group the n index is the slow one and the row inside the group the fast one (keeps the weight
    panel of one n resident in L2 while ``group_rows`` activations panels reuse it).
    """
    ids = np.arange(P, dtype=np.int64)
    if not group_rows:
        return ids.astype(np.int32)
    m, n = ids // tn1, ids % tn1
    key = ((m // group_rows) * tn1 + n) * group_rows + m % group_rows
    return np.argsort(key, kind="stable").astype(np.int32)


class QueueSim:
    """Sequential model of one producer->consumer link (reference csrc/ctapp.cuh:51-69).

    ``finish(tile)`` is what a producer CTA does after its tile has landed in the consumer's memory:
    walk the tile's CSR row, decrement each listed counter, and when a counter reaches zero publish the
    now-ready consumer work: in row-panel mode the ``tiles_n2`` ids ``c*tiles_n2 + j`` in ascending j on
    consecutive queue slots reserved with one fetch-add, in tile mode the single id ``c``.
    """

    def __init__(self, dep_offsets, dep_consumers, scoreboard, n_consumer_tiles, tiles_n2, rowpanel):
        self.off = np.asarray(dep_offsets)
        self.cons = np.asarray(dep_consumers)
        self.sb = np.array(scoreboard, dtype=np.int64, copy=True)
        self.cap = int(n_consumer_tiles)
        self.entries = np.full(self.cap, EMPTY, dtype=np.int64)
        self.tail = 0
        self.tiles_n2 = int(tiles_n2)
        self.rowpanel = bool(rowpanel)

    def finish(self, tile):
        for i in range(self.off[tile], self.off[tile + 1]):
            c = int(self.cons[i])
            k = c * PAD if self.rowpanel else c
            old = self.sb[k]
            self.sb[k] = old - 1
            if old != 1:
                continue
            if self.rowpanel:
                base = self.tail
                self.tail += self.tiles_n2
                for j in range(self.tiles_n2):
                    self.entries[(base + j) % self.cap] = c * self.tiles_n2 + j
            else:
                slot = self.tail
                self.tail += 1
                self.entries[slot % self.cap] = c


def simulate_link(M, N1, N2, BM1, BN1, BM2, BN2, rowpanel=True, group_rows=0, order=None):
    """Run the protocol with the producer finishing its tiles strictly in queue order (a one-CTA
    producer).  Returns (entries, tail, final scoreboard): the bit-exact readiness order a serialised
    device run must reproduce."""
    off, cons, sb = build_deps(M, N1, N2, BM1, BN1, BM2, BN2, rowpanel)
    tn1 = cdiv(N1, BN1)
    P = cdiv(M, BM1) * tn1
    C = cdiv(M, BM2) * cdiv(N2, BN2)
    q = QueueSim(off, cons, sb, C, cdiv(N2, BN2), rowpanel)
    for t in (producer_order(P, tn1, group_rows) if order is None else order):
        q.finish(int(t))
    return q.entries.astype(np.int32), q.tail, q.sb.astype(np.int32)


def simulate_kchunk_link(order1, tn1, order2, tn2, chunks, run_id=1):
    """Sequential model of one link with k-chunk dependencies (value flags per producer tile instead of a scoreboard and a
    queue): the producer finishes its tiles in ``order1`` (ids m * tn1 + n) and raises flag[m, n] = run_id; consumer tile
    m * tn2 + n2 may load k-chunk c once flag[m, c] is up.  Returns (flags after the run, for every consumer tile in
    ``order2`` the number of producer tiles that must have finished before it can complete).  The second array is the
    readiness order of a serialised device run; a consumer that walks ``order2`` never waits for a tile that a producer
    walking ``order1`` has not been able to start (there is no back edge), so the pair cannot deadlock."""
    order1, order2 = np.asarray(order1).astype(np.int64), np.asarray(order2).astype(np.int64)
    tm = order1.size // tn1
    done_at = np.empty(order1.size, dtype=np.int64)
    done_at[order1] = np.arange(1, order1.size + 1)
    done_at = done_at.reshape(tm, tn1)
    assert chunks <= tn1
    need = np.array([done_at[t // tn2, :chunks].max() for t in order2], dtype=np.int64)
    flags = np.full((tm, tn1), run_id, dtype=np.int32)
    return flags, need


def check_link_invariants(entries, tail, scoreboard, n_consumer_tiles, tiles_n2, rowpanel):
    """Order-independent invariants every (concurrent) run must satisfy.  Returns a list of violations."""
    bad = []
    e = np.asarray(entries).astype(np.int64)
    if int(tail) != n_consumer_tiles:
        bad.append(f"tail {int(tail)} != {n_consumer_tiles}")
    if np.any(np.asarray(scoreboard) != 0):
        bad.append("scoreboard not drained to zero")
    if sorted(e.tolist()) != list(range(n_consumer_tiles)):
        bad.append("queue is not a permutation of the consumer tile ids")
    elif rowpanel:
        blocks = e.reshape(-1, tiles_n2)
        if np.any(blocks[:, 0] % tiles_n2 != 0) or np.any(np.diff(blocks, axis=1) != 1):
            bad.append("a row panel's ids are not contiguous and ascending")
    return bad


# --------------------------------------------------------------------------------------------------
# arithmetic
def make_chain_inputs(M, K, widths, seed=0):
    """Seeded synthetic inputs of the chain benchmark: X ~ N(0,1), W_l ~ N(0, 1/fan_in), bf16.
    Generated on the CPU so the device path and the oracle see identical bits."""
    import torch
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(M, K, generator=g).to(torch.bfloat16)
    Ws, fan_in = [], K
    for n in widths:
        Ws.append((torch.randn(n, fan_in, generator=g) / fan_in ** 0.5).to(torch.bfloat16))
        fan_in = n
    return X, Ws


def chain_reference(X, Ws, keep=False):
    """Y_l = bf16( fp32( Y_{l-1} ) @ fp32( W_l )^T ), no activation (reference tests/test_ctapp.py:33 with the
    inter-stage tensor in bf16 as every implementation stores it).  Returns the last Y (bf16) or all."""
    import torch
    ys, y = [], X
    with torch.no_grad():
        for W in Ws:
            y = (y.float() @ W.float().t()).to(torch.bfloat16)
            ys.append(y)
    return ys if keep else y


def error_stats(got, ref):
    """(max relative error, mean abs error) after normalising by the RMS of the reference: the
    acceptance metric is max <= 2e-2 and mean <= 1e-3.  The max term uses |ref| clamped from below by
    the RMS so that near-zero outputs do not blow the ratio up."""
    import torch
    g, r = got.float(), ref.float()
    rms = r.pow(2).mean().sqrt().clamp_min(1e-30)
    d = (g - r).abs()
    return float((d / r.abs().clamp_min(rms)).max()), float(d.mean() / rms)
