"""Layer-per-GPU GEMM chain with CTA-level pipelining (mirrors reference ctapp/pipeline.py).

``build_deps`` builds the dependency CSR and the scoreboard; ``Pipeline`` is the reference's 2-GPU, 2-layer object with
the same constructor, attributes and methods; ``Chain`` generalises it to any number of stages driven from one
process; ``ChainStage`` is one stage owned by one process (one process per GPU), wired to its neighbours through
IPC-mapped buffers.
"""
from __future__ import annotations

import torch

from ctapp.ext import check_status, load, new_status

EMPTY = -1


def build_deps(M, N1, N2, BM1, BN1, BM2, BN2, rowpanel=True):
    """CSR dependency array over producer tiles (row-major ids m1 * tn1 + n1) and the consumer scoreboard's initial
    values, as int32 CPU tensors ``(dep_offsets, dep_consumers, init)``.

    rowpanel=True: one counter per consumer row panel, stored 32 ints apart (one 128-byte line each); the consumers of a
    producer tile are the row panels its rows intersect.  rowpanel=False: one counter per consumer tile (m2 * tn2 + n2).
    Same results as reference ctapp/pipeline.py:7-31.
    """
    tm1, tn1 = -(-M // BM1), -(-N1 // BN1)
    tm2, tn2 = -(-M // BM2), -(-N2 // BN2)
    m1 = torch.arange(tm1, dtype=torch.int64)
    first = m1 * BM1
    last = torch.minimum((m1 + 1) * BM1, torch.tensor(M)) - 1
    lo, hi = first // BM2, last // BM2
    width = 1 if rowpanel else tn2
    per_tile = ((hi - lo + 1) * width).repeat_interleave(tn1)           # out-degree of every producer tile
    offsets = torch.zeros(tm1 * tn1 + 1, dtype=torch.int64)
    torch.cumsum(per_tile, 0, out=offsets[1:])
    nnz = int(offsets[-1])
    owner = torch.repeat_interleave(torch.arange(tm1 * tn1), per_tile)  # producer tile of every CSR slot
    k = torch.arange(nnz) - offsets[owner]                              # position inside the tile's CSR row
    panel = lo[owner // tn1] + k // width
    consumers = panel if rowpanel else panel * tn2 + k % width
    counts = torch.bincount(consumers, minlength=tm2 if rowpanel else tm2 * tn2)
    if rowpanel:
        init = torch.zeros(tm2 * 32, dtype=torch.int64)
        init[::32] = counts
    else:
        init = counts
    return offsets.int(), consumers.int(), init.int()


def ramp_groups(tm, peak=8):
    """Group sizes 1, 1, 2, 4, ..., peak, ..., 4, 2, 1, 1 summing to ``tm`` tile rows: small groups first so that the first
    row panels complete (and the next stage starts) early, large groups in the middle for L2 reuse of the weight panels,
    small groups last so that little work is left for the next stage once this one has finished."""
    up, g = [1, 1], 2
    while g < peak:
        up.append(g); g *= 2
    sizes = []
    head, tail = [], []
    left = tm
    for a in up:                       # take the ramp from both ends while rows remain
        for side in (head, tail):
            if left >= a and left - a >= 0 and (left - a >= peak or left <= 2 * sum(up)):
                side.append(a); left -= a
            if left == 0:
                break
        if left == 0:
            break
    while left > 0:
        a = min(peak, left)
        sizes.append(a); left -= a
    return head + sizes + tail[::-1]


def head_groups(tm, peak=8):
    """Group sizes 2, 4, ..., then ``peak`` for the rest of ``tm`` tile rows.  The first wave of a GEMM covers a little more than
    two tile rows whatever the order, so a first group of two completes as early as anything can (a short fill for the next
    stage), and everything after the ramp keeps the L2 reuse of large groups.  For chains whose steps overlap, where what
    is left at the end of a step never idles the next stage."""
    sizes, g, left = [], 2, tm
    while left > 0:
        a = min(g, peak, left)
        sizes.append(a); left -= a
        g *= 2
    return sizes


def _group_sizes(group_rows, tm):
    """List of group sizes for the named or listed variable-group orders."""
    if group_rows == "ramp":
        return ramp_groups(tm)
    if group_rows == "head":
        return head_groups(tm)
    return list(group_rows)


def producer_order(P, tn1, group_rows):
    """Tile ids in the order the first stage works through them: groups of tile rows, n-major inside a group (reference
    ctapp/pipeline.py:48-51 for a constant group size).  ``group_rows``: 0 = ascending ids; an int = constant group size;
    "ramp" (``ramp_groups``), "head" (``head_groups``) or a list of group sizes = variable groups."""
    if not group_rows:
        return torch.arange(P, dtype=torch.int32)
    tm = P // tn1
    if isinstance(group_rows, int):
        t = torch.arange(P)
        m, n = t // tn1, t % tn1
        return torch.argsort(((m // group_rows) * tn1 + n) * group_rows + m % group_rows, stable=True).int()
    sizes = _group_sizes(group_rows, tm)
    assert sum(sizes) == tm and all(s > 0 for s in sizes), (sizes, tm)
    out, m0 = [], 0
    for g in sizes:
        rows = torch.arange(m0, m0 + g)
        out.append((rows[None, :] * tn1 + torch.arange(tn1)[:, None]).reshape(-1))   # n-major: for each n, the g rows
        m0 += g
    return torch.cat(out).int()


def _tile(ext, cfg):
    s = ext.config_info(cfg).split("tile ")[1].split("x")
    return int(s[0]), int(s[1])


def pop_slots(ntiles, tn, group):
    """Queue slot read by the i-th pop of a consuming stage (host model of the kernel's ``queue_slot``): windows of published
    row panels, n-tile major inside a window.  ``group``: an int = windows of that many panels (the last one takes the panels
    that are left; <= 1: queue order), or a list of window sizes summing to the number of row panels."""
    idx = torch.arange(ntiles)
    if isinstance(group, int):
        if group <= 1:
            return idx.int()
        tm = ntiles // tn
        group = [group] * (tm // group) + ([tm % group] if tm % group else [])
    sizes = torch.tensor(list(group))
    assert int(sizes.sum()) * tn == ntiles and bool((sizes > 0).all()), (group, ntiles, tn)
    first = torch.cumsum(sizes, 0) - sizes
    w = torch.repeat_interleave(torch.arange(len(sizes)), sizes * tn)      # window of every pop
    base, gw = first[w] * tn, sizes[w]
    r = idx - base
    return (base + (r % gw) * tn + r // gw).int()


def consumer_window(group_rows, rowpanel, bm_prev, bm, tm=0):
    """How a consuming stage pops its queue, given the order its producer works in: an int (constant windows of that many of
    this stage's row panels; 0 = queue order) or, for a producer with varying groups ("ramp" or a list), the list of window
    sizes.  The windows are the row panels the producer finishes together."""
    if not rowpanel or not group_rows:
        return 0
    if isinstance(group_rows, int):
        g = group_rows * bm_prev // bm
        return g if g > 1 else 0
    if bm_prev != bm:
        return 0
    return _group_sizes(group_rows, tm)


def _window_args(win, dev):
    """(src_group, src_windows tensor or None) for the bindings."""
    if isinstance(win, int):
        return win, None
    off = torch.zeros(len(win) + 1, dtype=torch.int32)
    off[1:] = torch.cumsum(torch.tensor(win), 0)
    return 0, off.to(dev)


class Pipeline:
    """2-layer CTA-pipelined run: the producer GEMM on devA stores Y1 into devB's memory tile by tile, the consumer GEMM
    on devB starts each tile as soon as the row panel it reads is complete.  Same constructor, attributes and methods
    as reference ctapp/pipeline.py:34-81; a two-stage ``Chain`` underneath.  devA == devB runs both stages on one GPU,
    one after the other on the same stream."""

    def __init__(self, M, K, N1, N2, cfg1, cfg2, devA=0, devB=1, skip_wait=0, fence=0, group_rows=0, scoreboard="rowpanel"):
        assert scoreboard in ("rowpanel", "tile", "kchunk")
        ch = Chain(M, K, [N1, N2], [devA, devB], cfg=[cfg1, cfg2], group_rows=group_rows, scoreboard=scoreboard,
                   fence=fence, skip_wait=skip_wait)
        self.chain, self.ext = ch, ch.ext
        self.M, self.cfg1, self.cfg2, self.skip_wait, self.fence, self.rowpanel = M, cfg1, cfg2, skip_wait, fence, ch.rowpanel
        self.a, self.b = ch.devs
        self.tn1, self.tn2 = ch.tn
        self.src_a, self.src_b = ch.entries
        self.head_a, self.head_b = ch.head
        self.tail_a, self.tail_b = ch.tail
        self.dep_off, self.dep_cons, self.sb, self.sb_pristine = ch.dep_off[0], ch.dep_cons[0], ch.sb[0], ch.sb_pristine[0]
        self.Y1, self.Y2 = ch.Y
        self.status_a, self.status_b = ch.status

    def tile(self, cfg):
        return _tile(self.ext, cfg)

    def reset(self):
        self.chain.reset()

    def run(self, X, W1, W2):
        return self.chain.run(X, [W1, W2])

    def check(self):
        """Synchronise both devices and raise if a device-side wait gave up."""
        self.chain.check()


class Chain:
    """N-stage chain driven from one process: stage g runs on ``devices[g]`` with weight W_g (N_g, N_{g-1}); its output
    tiles land in the memory of ``devices[g+1]`` and are announced in that GPU's work queue.  Repeated devices are
    allowed (stages then run back to back on that GPU's stream).

    scoreboard: "rowpanel" / "tile" = the reference's dependency CSR + scoreboard + work queue (a consumer tile is released
    when its whole row panel, or tile set, is complete).  "kchunk" = value flags per producer tile instead: every stage walks
    its own fixed tile order (``group_rows`` for all of them) and a consuming tile waits, k-chunk by k-chunk, for the flag
    of the producer tile that holds those columns of its input rows, so its main loop streams behind the producer while both
    keep an L2-friendly order.  Needs tiles of the same height on both sides of every link."""

    def __init__(self, M, K, widths, devices, cfg=3, group_rows=8, scoreboard="rowpanel", fence=1, skip_wait=0, sms=0, stamps=False,
                 consumer_group="auto"):
        self.ext = load()
        self.sms = sms
        self.stamps = None       # per stage: 8 int64 per CTA (ctapp.timeline reads them), when ``stamps`` is set
        self.M, self.K, self.widths, self.fence, self.skip_wait = M, K, list(widths), fence, skip_wait
        self.cfg = list(cfg) if isinstance(cfg, (list, tuple)) else [cfg] * len(self.widths)
        self.devs = [torch.device("cuda", d) for d in devices]
        assert len(self.devs) == len(self.widths) >= 1
        self.rowpanel = int(scoreboard == "rowpanel")
        self.kchunk = scoreboard == "kchunk"
        self.run_id = 0          # k-chunk flags carry the run's number: they only ever grow and are never reset
        for a, b in zip(devices[:-1], devices[1:]):
            if a != b:
                self.ext.enable_peer_access(a, b); self.ext.enable_peer_access(b, a)
        for d in set(devices):
            self.ext.preload(d)
        tiles = [_tile(self.ext, c) for c in self.cfg]
        i32 = dict(dtype=torch.int32)
        L = len(self.widths)
        wins = [0] + [0 if self.kchunk else consumer_window(group_rows, self.rowpanel, tiles[g - 1][0], tiles[g][0], -(-M // tiles[g][0]))
                      if consumer_group == "auto" else consumer_group for g in range(1, L)]
        if self.kchunk:
            assert all(t[0] == tiles[0][0] for t in tiles), f"k-chunk dependencies need tiles of one height on every stage, got {tiles}"
        self.src_group, self.src_windows = zip(*[_window_args(w, self.devs[g]) for g, w in enumerate(wins)])
        self.tn = [-(-n // t[1]) for n, t in zip(self.widths, tiles)]
        self.ntiles = [-(-M // t[0]) * tn for t, tn in zip(tiles, self.tn)]
        self.entries, self.head, self.tail, self.Y, self.status = [], [], [], [], []
        self.dep_off, self.dep_cons, self.sb, self.sb_pristine = [], [], [], []
        # k-chunk mode: chunk[g] = flags of stage g's INPUT rows, in stage g's memory, one per tile of stage g-1
        self.chunk = [None] + [torch.zeros(-(-M // tiles[g][0]), self.tn[g - 1], device=self.devs[g], **i32) if self.kchunk else None
                               for g in range(1, L)]
        self.chunk_kblocks = [0] + [tiles[g - 1][1] // 64 for g in range(1, L)]
        for g in range(L):
            dev = self.devs[g]
            if g == 0 or self.kchunk:
                self.entries.append(producer_order(self.ntiles[g], self.tn[g], group_rows).to(dev))     # a fixed order, always full
                self.tail.append(torch.full((1,), self.ntiles[g], device=dev, **i32))
            else:
                self.entries.append(torch.full((self.ntiles[g],), EMPTY, device=dev, **i32))
                self.tail.append(torch.zeros(1, device=dev, **i32))
            self.head.append(torch.zeros(1, device=dev, **i32))
            self.status.append(new_status(dev))
            if stamps:
                self.stamps = (self.stamps or []) + [torch.zeros(256 * 8, dtype=torch.int64, device=dev)]
            out_dev = self.devs[g + 1] if g + 1 < L else dev
            self.Y.append(torch.empty(M, self.widths[g], device=out_dev, dtype=torch.bfloat16))
            if g + 1 < L and not self.kchunk:
                off, cons, sb = build_deps(M, self.widths[g], self.widths[g + 1], *tiles[g], *tiles[g + 1], bool(self.rowpanel))
                self.dep_off.append(off.to(dev)); self.dep_cons.append(cons.to(dev))
                self.sb_pristine.append(sb.to(dev)); self.sb.append(sb.to(dev).clone())
            else:
                self.dep_off.append(None); self.dep_cons.append(None); self.sb.append(None); self.sb_pristine.append(None)

    def reset(self):
        """One reset kernel per stage (queue entries = -1, head = tail = 0, scoreboard restored); stage g may write into
        stage g+1's memory only after that stage's reset, which a stream event orders across GPUs."""
        L = len(self.widths)
        evs = [None] * L
        self.run_id += 1
        for g in range(L):
            with torch.cuda.device(self.devs[g]):
                self.ext.chain_reset(None if g == 0 or self.kchunk else self.entries[g], self.head[g], self.tail[g], self.sb[g], self.sb_pristine[g])
                if g > 0 and self.devs[g - 1] != self.devs[g]:
                    evs[g] = torch.cuda.Event(); evs[g].record()
        for g in range(L - 1):
            if evs[g + 1] is not None:
                torch.cuda.current_stream(self.devs[g]).wait_event(evs[g + 1])

    def enqueue(self, X, Ws):
        L = len(self.widths)
        for g in range(L):
            with torch.cuda.device(self.devs[g]):
                inp = X if g == 0 else self.Y[g - 1]
                last = g + 1 == L
                queued = not last and not self.kchunk        # publish into the next stage's work queue
                self.ext.ctapp_gemm(inp, Ws[g], self.Y[g], self.cfg[g], self.entries[g], self.head[g], self.tail[g],
                                    self.dep_off[g], self.dep_cons[g], self.sb[g],
                                    self.entries[g + 1] if queued else None, self.head[g + 1] if queued else None,
                                    self.tail[g + 1] if queued else None, self.tn[g], self.skip_wait if g > 0 else 0, self.fence,
                                    tiles_n2=self.tn[g + 1] if queued else 0, rowpanel=self.rowpanel, status=self.status[g], sms=self.sms,
                                    stamps=self.stamps[g] if self.stamps else None, src_group=self.src_group[g], src_windows=self.src_windows[g],
                                    chunk_dst=None if last else self.chunk[g + 1], chunk_src=self.chunk[g], chunk_kblocks=self.chunk_kblocks[g],
                                    chunk_value=self.run_id)
        return self.Y[-1]

    def run(self, X, Ws):
        self.reset()
        return self.enqueue(X, Ws)

    def check(self):
        for d in self.devs:
            torch.cuda.synchronize(d)
        for g, s in enumerate(self.status):
            check_status(s, f"chain stage {g}")


def stage_plan(M, K, widths, rank, tile=(128, 256)):
    """Sizes of stage ``rank`` of an N-stage chain and of the link to its successor: a pure function every rank evaluates
    for itself and for its neighbours (the queue a stage publishes into must have exactly the successor's tile count)."""
    BM, BN = tile
    world = len(widths)
    ins = [K] + list(widths[:-1])
    tm = -(-M // BM)
    tn = -(-widths[rank] // BN)
    plan = {"rank": rank, "k_in": ins[rank], "n_out": widths[rank], "tiles_m": tm, "tiles_n": tn, "ntiles": tm * tn,
            "first": rank == 0, "last": rank == world - 1}
    if rank + 1 < world:
        tn2 = -(-widths[rank + 1] // BN)
        plan.update(tiles_n2=tn2, dst_cap=tm * tn2, dst_rows=M, dst_cols=widths[rank])
    else:
        plan.update(tiles_n2=0, dst_cap=0, dst_rows=0, dst_cols=0)
    return plan


class ChainStage:
    """One stage of an N-stage chain, owned by one process (one process per GPU, ``torch.distributed`` initialised).

    Rank g holds W_g and computes Y_g = Y_{g-1} W_g^T.  Its input buffer and its work queue live in its own memory and are
    mapped into rank g-1, whose GEMM epilogue stores finished tiles straight into that buffer and publishes completed row
    panels in that queue.  No collective is on the data path.  Re-running needs no host synchronisation between ranks.

    Every link (input buffer, queue, ready flag) exists twice, used by odd and even steps in turn, so that consecutive
    steps overlap the way batches stream through a layer pipeline: while this rank still works on step e out of one set,
    rank g-1 already stores step e+1 into the other.  ``step(e)`` first resets the set of step e+1 (free since this rank's
    GEMM of step e-1, which precedes it in stream order) and raises that set's ready flag in rank g-1's memory to e+1;
    rank g-1's epilogue waits for that value before its first store of step e+1.  At most two steps are in flight per link.

    scoreboard="kchunk": value flags per tile of rank g-1 instead of dependency CSR, scoreboard and queue (see ``Chain``): every
    rank walks its own fixed grouped order; rank g-1's epilogue raises flag[set][m][n] = step number in rank g's memory, and rank
    g's tiles wait k-chunk by k-chunk.  The flags only grow, so a set's flags of step e - 2 never satisfy step e and nothing but
    the queue head is reset; the ready flag still keeps rank g-1 from overwriting rows that step e - 2 is reading.
    """

    def __init__(self, M, K, widths, rank, world, device, group=None, cfg=3, group_rows=8, scoreboard="rowpanel", consumer_group="auto"):
        from ctapp.symm import symm_empty, view_ptr
        assert len(widths) == world
        self.ext = load()
        self.M, self.rank, self.world, self.cfg = M, rank, world, cfg
        self.dev = device if isinstance(device, torch.device) else torch.device("cuda", device)
        assert scoreboard in ("rowpanel", "tile", "kchunk")
        self.rowpanel = int(scoreboard == "rowpanel")
        self.kchunk = scoreboard == "kchunk"
        self.ext.preload(self.dev.index)
        BM, BN = _tile(self.ext, cfg)
        win = 0 if rank == 0 or self.kchunk else (consumer_window(group_rows, self.rowpanel, BM, BM, -(-M // BM)) if consumer_group == "auto" else consumer_group)
        self.src_group, self.src_windows = _window_args(win, self.dev)
        plan = stage_plan(M, K, widths, rank, (BM, BN))
        tm = plan["tiles_m"]
        self.k_in, self.n_out, self.tn, self.ntiles = plan["k_in"], plan["n_out"], plan["tiles_n"], plan["ntiles"]
        first, last = plan["first"], plan["last"]
        # symmetric buffers (collective, same order on every rank); leading dimension 2 = the set of odd / even steps
        self.Yin2, h_y = symm_empty((2, M, self.k_in) if not first else (8,), torch.bfloat16, self.dev, group, rank)
        self.entries_sym, h_e = symm_empty((2, self.ntiles), torch.int32, self.dev, group, rank)
        self.ctl, h_c = symm_empty((2, 4), torch.int32, self.dev, group, rank)       # per set: [head, tail, ready, -]
        self._hdls = (h_y, h_e, h_c)   # all three arrive zero-filled; peers may write flags into ctl from here on
        tn_in = 1 if first else -(-self.k_in // BN)          # tiles per row of the rank before this one (same tile on every rank)
        self.chunk2 = self.dst_chunk2 = None
        if self.kchunk:                                         # collective like the three above, zero-filled: step numbers start at 1
            self.chunk2, h_f = symm_empty((2, tm, tn_in), torch.int32, self.dev, group, rank)
            self._hdls += (h_f,)
            self.chunk_kblocks = BN // 64
        if first or self.kchunk:
            self.entries0 = producer_order(self.ntiles, self.tn, group_rows).to(self.dev)
            self.ctl[:, 1] = self.ntiles
        else:
            self.entries_sym.fill_(EMPTY)
        self.status = new_status(self.dev)
        self.epoch = 0
        if not last:
            n_next = widths[rank + 1]
            tn2 = -(-n_next // BN)
            self.tn2 = tn2
            if self.kchunk:
                self.dep_off = self.dep_cons = self.sb = self.sb_pristine = None
                self.dst_chunk2 = view_ptr(h_f.buffer_ptrs[rank + 1], (2, tm, self.tn), torch.int32, self.dev)
            else:
                off, cons, sb = build_deps(M, self.n_out, n_next, BM, BN, BM, BN, bool(self.rowpanel))
                self.dep_off, self.dep_cons = off.to(self.dev), cons.to(self.dev)
                self.sb_pristine = sb.to(self.dev); self.sb = self.sb_pristine.clone()
            nxt = rank + 1
            self.Yout2 = view_ptr(h_y.buffer_ptrs[nxt], (2, M, self.n_out), torch.bfloat16, self.dev)
            self.dst_entries2 = view_ptr(h_e.buffer_ptrs[nxt], (2, tm * tn2), torch.int32, self.dev)
            self.dst_ctl2 = view_ptr(h_c.buffer_ptrs[nxt], (2, 4), torch.int32, self.dev)
        else:
            self.tn2 = 0
            self.dep_off = self.dep_cons = self.sb = self.sb_pristine = None
            self.Yout2 = torch.empty(1, M, self.n_out, dtype=torch.bfloat16, device=self.dev)
            self.dst_entries2 = self.dst_ctl2 = None
        self.up_ctl2 = None if first else view_ptr(h_c.buffer_ptrs[rank - 1], (2, 4), torch.int32, self.dev)
        self._reset_set(1)   # step 1 runs out of set 1
        torch.cuda.synchronize(self.dev)

    def _queue(self, s):
        """(entries, head, tail) this rank's GEMM pops in a step of set ``s``; rank 0 (with k-chunk flags: every rank) pops its
        fixed grouped order."""
        if self.rank == 0:
            return self.entries0, self.ctl[0, 0:1], self.ctl[0, 1:2]
        if self.kchunk:
            return self.entries0, self.ctl[s, 0:1], self.ctl[s, 1:2]
        return self.entries_sym[s], self.ctl[s, 0:1], self.ctl[s, 1:2]

    def _reset_set(self, e):
        """Reset this rank's queue of set e % 2 for step ``e`` and tell rank g-1 it may store that step; restores the
        scoreboard of the outgoing link on the way (the GEMM enqueued next is its only user)."""
        first = self.rank == 0
        s = e & 1
        entries, head, tail = self._queue(s)
        with torch.cuda.device(self.dev):
            self.ext.chain_reset(None if first or self.kchunk else entries, head, tail, self.sb, self.sb_pristine,
                                 ready_flag=None if first else self.up_ctl2[s, 2:3], ready_value=e)

    @property
    def Yin(self):
        """Input buffer of the step enqueued last (rank 0 has none)."""
        return None if self.rank == 0 else self.Yin2[self.epoch & 1]

    @property
    def Yout(self):
        """Where the step enqueued last put its output: the next rank's input buffer of that step, or a local tensor."""
        return self.Yout2[(self.epoch & 1) if self.rank + 1 < self.world else 0]

    def step(self, W, X=None):
        """Enqueue one run of this stage.  Rank 0 passes the chain's input X; the other ranks read their input buffer."""
        self.epoch += 1
        e = self.epoch
        s = e & 1
        first, last = self.rank == 0, self.rank == self.world - 1
        self._reset_set(e + 1)
        entries, head, tail = self._queue(s)
        with torch.cuda.device(self.dev):
            inp = X if first else self.Yin2[s]
            out = self.Yout2[0 if last else s]
            queued = not last and not self.kchunk
            self.ext.ctapp_gemm(inp, W, out, self.cfg, entries, head, tail, self.dep_off, self.dep_cons, self.sb,
                                self.dst_entries2[s] if queued else None, self.dst_ctl2[s, 0:1] if queued else None,
                                self.dst_ctl2[s, 1:2] if queued else None, self.tn, 0, 1, tiles_n2=self.tn2 if queued else 0, rowpanel=self.rowpanel,
                                status=self.status, dst_ready=None if last else self.ctl[s, 2:3], ready_value=e, src_group=self.src_group, src_windows=self.src_windows,
                                chunk_dst=self.dst_chunk2[s] if self.kchunk and not last else None,
                                chunk_src=self.chunk2[s] if self.kchunk and not first else None,
                                chunk_kblocks=self.chunk_kblocks if self.kchunk else 0, chunk_value=e)
        return out

    def check(self):
        torch.cuda.synchronize(self.dev)
        check_status(self.status, f"chain stage {self.rank}")
