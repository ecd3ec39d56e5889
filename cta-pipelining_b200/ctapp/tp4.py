"""Tensor-parallel layer boundary  down-proj -> cross-rank sum + residual -> RMSNorm -> next projection  (mirrors
reference ctapp/tp4.py).

Per rank r of ``world`` (2, 4 or 8; 1 = one GPU talking to itself):
  h_r       (M, Kr)       K-shard of the FFN hidden
  Wdown_r   (n1, Kr)      W_down[:, r*Kr:(r+1)*Kr]
  Wqkv_r    (N2r, n1)     W_qkv[r*N2r:(r+1)*N2r] with the RMSNorm gamma folded in
  out_r     (M, N2r)      output column shard
The reduced residual stream x_new = resid + sum_r h_r Wdown_r^T is left in full on every rank (``x()``).

``CtappBoundary`` runs the panel-ownership protocol: rank r owns the 128-row panels m with m % world == r; every
producer GEMM stores tile (m, n) straight into the owner's inbox and raises a value flag there; the owner reducer sums
the ``world`` inbox slices + resid, pushes x and the row sums of squares to every rank and raises the panel flag; the
consumer GEMM waits per panel and scales its rows by rsqrt(rowss / n1 + eps).  The other classes are comparison
baselines with the same ``forward(h_r, resid)`` signature.
"""
from __future__ import annotations

import logging
import os

import torch
import torch.distributed as dist

from ctapp.ext import check_status, load_tp4, new_status
from ctapp.symm import LocalGroup, symm_empty

log = logging.getLogger("ctapp")

DTYPE = torch.bfloat16
EPS = 1e-5
N1 = 8192          # hidden size (down-proj N, RMSNorm width)
K_FFN = 28672
N2 = 10240         # fused QKV width


def _symm(shape, dtype, dev, group_name, rank=None, multicast=False):
    """(tensor, handle with ``buffer_ptrs`` / ``multicast_ptr``): reference ctapp/tp4.py:31-35."""
    return symm_empty(shape, dtype, dev, group_name, rank, multicast)


def shard_weights(Wdown, Wqkv, gamma, rank, world):
    """Full weights -> (Wdown_r, Wqkv_r unfolded, Wqkv_r with gamma folded), bf16 contiguous (reference ctapp/tp4.py:38-44)."""
    Kr, N2r = Wdown.shape[1] // world, Wqkv.shape[0] // world
    Wd = Wdown[:, rank * Kr:(rank + 1) * Kr].contiguous()
    Wq = Wqkv[rank * N2r:(rank + 1) * N2r].contiguous()
    return Wd, Wq, fold_gamma(Wq, gamma)


def rmsnorm_gamma(x, gamma, eps=EPS):
    """Eager, unfused: bf16(x * rsqrt(mean(x^2) + eps)) * gamma (reference ctapp/tp4.py:47-50)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * gamma


def fold_gamma(Wq, gamma):
    """RMSNorm gamma folded into the weight's columns: bf16(fp32(Wq) * fp32(gamma)[None, :]) (reference ctapp/tp4.py:53-56)."""
    return (Wq.float() * gamma.float()[None, :]).to(DTYPE).contiguous()


def interleave_gate_up(W, block=128):
    """(2 I, K) weight with the gate rows first and the up rows second -> the same rows in blocks of ``block``: gate rows
    0..block-1, up rows 0..block-1, gate rows block..2 block-1, ...  A 256-column output tile of the consumer GEMM then
    holds 128 gate columns and their 128 up columns, which is what its activation epilogue (``act``) combines."""
    two_i, K = W.shape
    I = two_i // 2
    assert two_i % 2 == 0 and I % block == 0, (W.shape, block)
    return torch.stack((W[:I].view(I // block, block, K), W[I:].view(I // block, block, K)), dim=1).reshape(two_i, K).contiguous()


# --------------------------------------------------------------------------- CTA-pipelined boundary
class CtappBoundary:
    """CTA-pipelined boundary, panel-ownership protocol with unicast value flags (the reference's protocol "v5",
    ctapp/tp4.py:60-504), for world in {1, 2, 4, 8}.

    Per forward: ``tp4_step`` (epoch += 1, zero the per-step accumulators) -> producer GEMM mode 7 on ``SMs - R`` SMs ||
    owner reducer (``red_blocks`` CTAs of ``red_threads`` threads on a second stream) -> consumer GEMM mode 5 on
    ``SMs - R`` SMs.  All flags are epoch values, so one instance sized ``max_M`` serves every M <= max_M with
    M % 128 == 0; ``out`` and ``x()`` are views of the first M rows.

    protocol: "v5" (default here) = unicast pushes; True / "v3" = NVLS variant: the same panel-ownership protocol, but the owner
    reducer pushes x, the row sums and the panel flags with ``multimem.st`` on multicast addresses, so each row leaves the
    owner once and the NVSwitch replicates it (needs one process per GPU, >= 2 ranks, torch symmetric memory with multicast;
    falls back to unicast with a warning otherwise).  False = the two GEMMs alone (no exchange, no residual): the floor the
    protocol is measured against.
    fusion: "none" = reducer on a side stream, consumer after the producer in stream order;
            "pdl"  = as "none" and the consumer is launched as the producer's programmatic dependent, so its CTAs start
                     as producer CTAs retire (the per-panel flags carry the data dependency);
            "serial" = step, producer, reducer, consumer on one stream, nothing concurrent on this GPU (used where a
                     single GPU plays every rank).
    use_graph: forwards are captured into CUDA graphs keyed by (parity, M); inputs are copied into static buffers
    before each replay (``graph_bind`` captures the caller's tensors instead).
    act: the consumer's weight is a gate/up projection with rows interleaved by ``interleave_gate_up``; its epilogue applies
    silu(gate) * up and ``out`` is (M, N2r / 2): the activation costs no pass over memory of its own.
    cta_pair: both GEMMs run as CTA pairs (``cta_group::2``, 256-row tiles; the protocol's unit stays the 128-row panel);
    False = one CTA per 128-row tile.
    ``group_name``: a torch.distributed group name (one process per GPU) or a ``ctapp.symm.LocalGroup`` (one process
    drives every rank's GPU).
    """

    def __init__(self, M, Kr, N2r, rank, world, group_name, device, resid=True, protocol="v5", use_graph=False, R=None,
                 qkv_raster=2, qkv_swizzle=1, max_M=None, down_raster=None, red_threads=1024, red_blocks=None, red_variant=1,
                 fusion="none", qkv_tile=256, role_rows=4, down_swizzle=1, pdl_trigger=None, trace=None, role_stages=0, steal=False,
                 down_tail="auto", graph_bind=False, n1=N1, eps=EPS, cta_pair=True, act=False):
        assert M % 128 == 0 and n1 % 256 == 0, (M, n1)
        assert not act or (cta_pair and qkv_tile == 256 and N2r % 256 == 0), "act needs the CTA-pair consumer and N2r % 256 == 0"
        self.act = int(bool(act))
        assert protocol in (True, False, "v3", "v5"), protocol
        assert world in (1, 2, 4, 8), f"world {world} is not supported"
        # True / "v3": NVLS variant -- the owner reducer pushes x, row sums and panel flags with multimem stores on multicast
        # addresses (replicated inside the NVSwitch); needs one process per GPU, world >= 2 and multicast support
        self.nvls = protocol in (True, "v3") and world >= 2 and not isinstance(group_name, LocalGroup)
        if protocol in (True, "v3") and not self.nvls:
            log.warning("ctapp: NVLS needs one process per GPU and at least 2 ranks; using unicast pushes")
        assert fusion in ("none", "pdl", "serial"), f"fusion {fusion!r} is not available in this build (none | pdl | serial)"
        assert red_variant in (1, 3), "reducer variants of this build: 1 = warp per unit (register loads), 3 = TMA-fed"
        assert qkv_tile in (256, 128)
        assert down_tail == "auto" or (isinstance(down_tail, int) and 0 <= down_tail <= n1 // 256), down_tail
        self.ext = load_tp4()
        self.M, self.Kr, self.N2r, self.rank, self.world = M, Kr, N2r, rank, world
        self.n1, self.eps, self.cta_pair = n1, eps, int(bool(cta_pair))
        self.dev = device if isinstance(device, torch.device) else torch.device("cuda", device)
        self.use_resid, self.protocol, self.use_graph, self.v5 = resid, bool(protocol), use_graph, bool(protocol)
        self.group = group_name
        self.R = R or (8 if world >= 4 else 4)   # measured on B200 at M=4096: TP2 best with 4, TP4 and TP8 with 8
        self.qkv_raster, self.qkv_swizzle, self.qkv_tile = qkv_raster, qkv_swizzle, qkv_tile
        self.nsm = torch.cuda.get_device_properties(self.dev).multi_processor_count
        self.sms = self.nsm - self.R
        self.qkv_sms = self.sms
        self.fusion, self.down_swizzle, self.down_tail, self.steal = fusion, down_swizzle, down_tail, bool(steal)
        self.down_raster = down_raster or 1
        self.red_threads, self.red_blocks, self.red_variant = red_threads, red_blocks or self.R, red_variant
        self.graph_bind = bool(graph_bind)
        self.pdl_trigger = (1 if fusion == "pdl" else 0) if pdl_trigger is None else int(pdl_trigger)
        self.trace = bool(int(os.environ.get("CTAPP_TRACE", "0"))) if trace is None else bool(trace)
        self.max_M = max_M = max_M or M
        assert max_M % 128 == 0 and M <= max_M, (M, max_M)
        dev, tn = self.dev, n1 // 256
        with torch.cuda.device(dev):
            self.ext.preload(dev.index)
            self.ppo = ppo = -(-(max_M // 128) // world)            # panels per owner (ceil)
            sy = lambda shape, dt, mc=False: _symm(shape, dt, dev, group_name, rank, mc and self.nvls)  # noqa: E731
            self.inbox, hi = sy((world, ppo * 128, n1), DTYPE)       # this rank's inbox; slot s = source rank s
            self.tile_flags, ht = sy((world, ppo, tn), torch.int32)
            self.panel_flag, hp = sy((max_M // 128,), torch.int32, True)
            self.rowss, hr = sy((2, max_M), torch.float32, True)     # by epoch parity
            self.xbuf, hx0 = sy((max_M, n1), DTYPE, True)
            self.xbuf1, hx1 = sy((max_M, n1), DTYPE, True)
            if self.nvls and not (hp.multicast_ptr and hr.multicast_ptr and hx0.multicast_ptr and hx1.multicast_ptr):
                log.warning("ctapp: no multicast address on this system; using unicast pushes")
                self.nvls = False
            self._x_mc = [hx0.multicast_ptr, hx1.multicast_ptr] if self.nvls else [0, 0]
            self._rowss_mc = [hr.multicast_ptr + par * max_M * 4 for par in (0, 1)] if self.nvls else [0, 0]
            self._pf_mc = hp.multicast_ptr if self.nvls else 0
            self._hdls = (hi, ht, hp, hr, hx0, hx1)
            self.xbufs = [self.xbuf, self.xbuf1]
            slot = ppo * 128 * n1 * 2                                 # bytes of one inbox slot
            self._dst_ptrs = [hi.buffer_ptrs[d] + rank * slot for d in range(world)]       # producer: my slot at every owner
            self._peer_tf = [ht.buffer_ptrs[d] for d in range(world)]
            self._inbox_local = [self.inbox.data_ptr() + s * slot for s in range(world)]   # reducer: my inbox, per source
            self._peer_x = [[hx0.buffer_ptrs[d] for d in range(world)], [hx1.buffer_ptrs[d] for d in range(world)]]
            self._peer_rowss = [[hr.buffer_ptrs[d] + par * max_M * 4 for d in range(world)] for par in (0, 1)]
            self._peer_pf = [hp.buffer_ptrs[d] for d in range(world)]
            self.rowss_local = torch.zeros(max_M, dtype=torch.float32, device=dev)
            self.panel_done = torch.zeros(max_M // 128, dtype=torch.int32, device=dev)
            self.role_ctr = torch.zeros(2, dtype=torch.int32, device=dev)
            self.status = new_status(dev)
            self.trace_down = torch.zeros(self.nsm * 8, dtype=torch.int64, device=dev)
            self.trace_qkv = torch.zeros(self.nsm * 8, dtype=torch.int64, device=dev)
            self.trace_red = torch.zeros(max_M // 128, dtype=torch.int64, device=dev)
            for t in (self.tile_flags, self.panel_flag, self.rowss):
                t.zero_()
            self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=dev)
            self.s_red = torch.cuda.Stream(device=dev)
            self.ev_start, self.ev_red = torch.cuda.Event(), torch.cuda.Event()
            torch.cuda.synchronize(dev)
            self._out_full = torch.empty(max_M, N2r // 2 if self.act else N2r, dtype=DTYPE, device=dev)
            self._floor_y = None
            self.h_static = torch.empty(max_M, Kr, dtype=DTYPE, device=dev) if use_graph and not graph_bind else None
            self.resid_static = torch.empty(max_M, n1, dtype=DTYPE, device=dev) if use_graph and resid and not graph_bind else None
        _group_barrier(group_name)
        self.out = self._out_full[:M]
        self.epoch = 0
        self._last_par, self._last_M = 0, M
        self.Wd = self.Wq = None
        self._graphs = {}
        self._warm = False
        self._warmed = True     # kernels are loaded by preload(); no warm-up launches are needed

    # ---- pieces of one forward
    def _tail(self, M):
        if self.down_tail != "auto":
            return self.down_tail
        if self.down_raster != 1 or self.down_swizzle != 1:
            return 0
        return min(16 if M // 128 >= 16 else 8, self.n1 // 256)

    def _tr(self, t):
        return t.data_ptr() if self.trace else 0

    def _reduce_v5(self, M, resid, parity):
        self.ext.tp4_reduce(M, self.rank, self.world, 0, self.down_raster, self.red_blocks, self.tile_flags, resid=resid,
                            peer_x=self._peer_x[parity], version=5, epoch_dev=self.epoch_dev, inbox_ptrs=self._inbox_local,
                            peer_rowss=self._peer_rowss[parity], peer_panel_flag=self._peer_pf, rowss_local=self.rowss_local,
                            panel_done=self.panel_done, panels_per_owner=self.ppo, threads=self.red_threads, variant=self.red_variant,
                            red_trace=self._tr(self.trace_red), unit_ctr=self.role_ctr[1:] if self.steal else 0,
                            tail_cols=self._tail(M), n1=self.n1, status=self.status, x_mc_ptr=self._x_mc[parity],
                            rowss_mc_ptr=self._rowss_mc[parity], panel_flag_mc_ptr=self._pf_mc)

    def _down_v5(self, h_r, Wd, M):
        self.ext.tp4_down(h_r, Wd, None, self.down_raster, self.down_swizzle, 7, self.rank, self.world, 0, sms=self.sms,
                          epoch_dev=self.epoch_dev, dst_ptrs=self._dst_ptrs, dst_rows=self.ppo * 128, peer_tile_flags=self._peer_tf,
                          panels_per_owner=self.ppo, pdl_trigger=self.pdl_trigger, trace=self._tr(self.trace_down),
                          tail_cols=self._tail(M), status=self.status, cta_pair=self.cta_pair)

    def _qkv_v5(self, Wq, M, parity):
        self.ext.tp4_qkv(self.xbufs[parity][:M], Wq, self._out_full[:M], self.qkv_raster, self.qkv_swizzle, 5, 0, self.panel_flag, 1,
                         self.rowss[parity], sms=self.qkv_sms, pdl=1 if self.fusion == "pdl" else 0, epoch_dev=self.epoch_dev,
                         tile=self.qkv_tile, trace=self._tr(self.trace_qkv), status=self.status, eps=self.eps, cta_pair=self.cta_pair, act=self.act)

    def _enqueue_v5(self, h_r, resid, parity, Wd, Wq, M):
        cur = torch.cuda.current_stream(self.dev)
        self.ext.tp4_step(self.epoch_dev, self.rowss_local, self.panel_done, M, self.role_ctr)
        if self.fusion == "serial":
            self._down_v5(h_r, Wd, M)
            self._reduce_v5(M, resid, parity)
            self._qkv_v5(Wq, M, parity)
            return
        self.ev_start.record(cur)
        self.s_red.wait_event(self.ev_start)
        with torch.cuda.stream(self.s_red):
            self._reduce_v5(M, resid, parity)
            self.ev_red.record(self.s_red)
        self._down_v5(h_r, Wd, M)
        self._qkv_v5(Wq, M, parity)
        cur.wait_event(self.ev_red)

    def _enqueue_floor(self, h_r, Wd, Wq, M):
        """The two GEMMs with the same SM split and tile orders, no exchange (reference ctapp/tp4.py:365-369)."""
        if self._floor_y is None:
            self._floor_y = torch.empty(self.max_M, self.n1, dtype=DTYPE, device=self.dev)
        self.ext.tp4_down(h_r, Wd, self._floor_y[:M], self.down_raster, self.down_swizzle, 0, self.rank, self.world, 0, sms=self.sms,
                          tail_cols=self._tail(M), cta_pair=self.cta_pair)
        self.ext.tp4_qkv(self._floor_y[:M], Wq, self._out_full[:M], self.qkv_raster, self.qkv_swizzle, 0, 0, sms=self.qkv_sms, tile=self.qkv_tile,
                         cta_pair=self.cta_pair, act=self.act)

    # ---- public API
    def warmup(self):
        """Kept for API compatibility: every kernel is loaded at construction (``ctapp_preload``), so nothing is launched."""
        self._warmed = True

    def _check_w(self, Wd, Wq):
        assert Wd.shape == (self.n1, self.Kr) and Wd.dtype == DTYPE and Wd.is_contiguous(), (Wd.shape, Wd.dtype)
        assert Wq.shape == (self.N2r, self.n1) and Wq.dtype == DTYPE and Wq.is_contiguous(), (Wq.shape, Wq.dtype)

    def set_weights(self, Wdown_r, Wqkv_r_folded):
        """Default weights (used when forward() gets none; baked into the graphs when use_graph)."""
        self._check_w(Wdown_r, Wqkv_r_folded)
        self.Wd, self.Wq = Wdown_r, Wqkv_r_folded

    def forward(self, h_r, resid=None, Wd=None, Wq=None):
        """Wd (n1, Kr) / Wq (N2r, n1, gamma folded): bf16 contiguous weights for this call (no copy; they must stay alive
        until the stream work finishes); default = those from set_weights.  Not supported with use_graph."""
        if self.use_graph:
            assert Wd is None and Wq is None, "per-call weights are not supported with use_graph"
        Wd = self.Wd if Wd is None else Wd
        Wq = self.Wq if Wq is None else Wq
        assert Wd is not None and Wq is not None, "no weights: call set_weights() or pass Wd/Wq"
        self._check_w(Wd, Wq)
        r = resid if self.use_resid else None
        M = h_r.shape[0]
        assert M % 128 == 0 and 0 < M <= self.max_M, (M, self.max_M)
        assert h_r.shape == (M, self.Kr) and h_r.dtype == DTYPE and h_r.is_contiguous(), (h_r.shape, h_r.dtype)
        if r is not None:
            assert r.shape == (M, self.n1) and r.dtype == DTYPE and r.is_contiguous(), (r.shape, r.dtype)
        self.out = self._out_full[:M]
        self._last_M = M
        with torch.cuda.device(self.dev):
            if not self.protocol:
                self._enqueue_floor(h_r, Wd, Wq, M)
                return self.out
            self.epoch += 1
            par = self.epoch & 1
            self._last_par = par
            if r is not None:
                assert r.data_ptr() != self.xbufs[par].data_ptr(), "resid aliases the x buffer written by this forward"
            if not self.use_graph:
                self._enqueue_v5(h_r, r, par, Wd, Wq, M)
                return self.out
            if self.graph_bind:
                hs, rs = h_r, r
                key = (par, M, h_r.data_ptr(), r.data_ptr() if r is not None else 0)
            else:
                self.h_static[:M].copy_(h_r)
                if r is not None:
                    self.resid_static[:M].copy_(r)
                hs = self.h_static[:M]
                rs = self.resid_static[:M] if r is not None else None
                key = (par, M)
            if not self._warm:               # un-captured first forward (the device epoch advances with the host epoch)
                self._warm = True
                self._enqueue_v5(hs, rs, par, Wd, Wq, M)
                return self.out
            g = self._graphs.get(key)
            if g is None:
                torch.cuda.synchronize(self.dev)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._enqueue_v5(hs, rs, par, Wd, Wq, M)
                self._graphs[key] = g
            g.replay()
            return self.out

    def x(self):
        """New residual (M, n1) of the most recent forward; valid until two forwards later (x is double-buffered)."""
        if not self.protocol:
            return self._floor_y[:self._last_M]
        return self.xbufs[self._last_par][:self._last_M]

    def check(self):
        """Synchronise this rank's device and raise if a device-side wait gave up."""
        torch.cuda.synchronize(self.dev)
        check_status(self.status, f"boundary rank {self.rank}")

    def trace_summary(self):
        """CTAPP_TRACE stamps of the most recent eager forward, in us relative to the first producer CTA's entry."""
        torch.cuda.synchronize(self.dev)
        td, tq = self.trace_down.view(-1, 8).cpu(), self.trace_qkv.view(-1, 8).cpu()
        td, tq = td[td[:, 0] > 0], tq[tq[:, 0] > 0]
        if td.shape[0] == 0:
            return {}
        t0 = int(td[:, 0].min())
        us = lambda v: (int(v) - t0) / 1e3  # noqa: E731
        d = {"prod_ctas": int(td.shape[0]), "prod_entry_max": us(td[:, 0].max()), "prod_first_tile_max": us(td[:, 1].max()),
             "prod_end_min": us(td[:, 7].min()), "prod_end_max": us(td[:, 7].max()), "cons_ctas": int(tq.shape[0])}
        P = self._last_M // 128
        tr = self.trace_red.cpu()[[m for m in range(P) if m % self.world == self.rank]]
        if tr.numel() and int(tr.min()) > 0:
            d["red_first_panel"], d["red_last_panel"] = us(tr.min()), us(tr.max())
        if tq.shape[0]:
            d["cons_entry_min"], d["cons_first_tile_min"] = us(tq[:, 0].min()), us(tq[:, 1].min())
            d["cons_end_max"] = us(tq[:, 7].max())
        return d


def forward_lockstep(bds, h_rs, resids, Wds, Wqs):
    """One forward of every rank of a ``LocalGroup`` from this process, phase by phase: all producers, then all owner
    reducers, then all consumers.  When several ranks share a GPU (one device playing all ranks) no kernel is ever
    launched before the kernels it waits for, so nothing waits on the device; with one GPU per rank the phases of different
    ranks still overlap across GPUs.  Returns the list of per-rank outputs."""
    outs = []
    for bd, h in zip(bds, h_rs):
        M = h.shape[0]
        bd.epoch += 1
        bd._last_par, bd._last_M = bd.epoch & 1, M
        bd.out = bd._out_full[:M]
        with torch.cuda.device(bd.dev):
            bd.ext.tp4_step(bd.epoch_dev, bd.rowss_local, bd.panel_done, M, bd.role_ctr)
    for bd, h, Wd in zip(bds, h_rs, Wds):
        with torch.cuda.device(bd.dev):
            bd._down_v5(h, Wd, h.shape[0])
    for bd, h, r in zip(bds, h_rs, resids):
        with torch.cuda.device(bd.dev):
            bd._reduce_v5(h.shape[0], r if bd.use_resid else None, bd._last_par)
    for bd, h, Wq in zip(bds, h_rs, Wqs):
        with torch.cuda.device(bd.dev):
            bd._qkv_v5(Wq, h.shape[0], bd._last_par)
        outs.append(bd.out)
    return outs


def _group_barrier(group):
    if isinstance(group, LocalGroup):
        group.barrier()
    elif dist.is_initialized():
        from ctapp.symm import _process_group
        pg = _process_group(group)
        if dist.get_world_size(pg) > 1:
            dist.barrier(group=pg)


class CtappBoundaryPool:
    """One boundary object shared by all layers (weights are passed per forward call).

    ``get(M)`` returns None when M is unsupported (M % 128 != 0, M < min_M or M > max_M): the caller uses its stock
    path.  Otherwise it returns the single instance sized ``max_M`` (value flags make it serve every M), creating it
    on first use.  Creation is COLLECTIVE (symmetric allocation + barrier): every rank must make its first valid
    ``get`` at the same point.  Same constructor as reference ctapp/tp4.py:507-554; ``protocol`` "v3" and "v5" both map
    to the unicast panel-ownership protocol here.
    """

    def __init__(self, Kr, N2r, rank, world, group_name, device, R=None, min_M=512, max_instances=4,
                 qkv_raster=2, qkv_swizzle=1, protocol="v5", max_M=8192, **v5kw):
        assert protocol in ("v3", "v5"), protocol
        self.Kr, self.N2r, self.rank, self.world, self.gn, self.dev = Kr, N2r, rank, world, group_name, device
        self.R, self.min_M, self.max_instances = R, min_M, max_instances
        self.qkv_raster, self.qkv_swizzle = qkv_raster, qkv_swizzle
        self.protocol, self.max_M = protocol, max_M
        self.v5kw = v5kw
        self._inst = {}

    def get(self, M):
        if M % 128 != 0 or M < self.min_M or M > self.max_M:
            return None
        bd = self._inst.get(self.max_M)
        if bd is None:
            bd = CtappBoundary(self.max_M, self.Kr, self.N2r, self.rank, self.world, self.gn, self.dev, R=self.R,
                               qkv_raster=self.qkv_raster, qkv_swizzle=self.qkv_swizzle, protocol=self.protocol, max_M=self.max_M, **self.v5kw)
            self._inst[self.max_M] = bd
        return bd


# --------------------------------------------------------------------------- baselines
class _Base:
    def __init__(self, M, rank, world, group_name, device, Wdown_r, Wqkv_r, gamma):
        self.M, self.rank, self.world, self.gn, self.dev = M, rank, world, group_name, device
        self.Wd, self.Wq, self.gamma = Wdown_r, Wqkv_r, gamma.to(DTYPE)
        self._x = None

    def x(self):
        return self._x

    def _post(self, y, resid):
        x = y + resid if resid is not None else y
        self._x = x
        return torch.mm(rmsnorm_gamma(x, self.gamma), self.Wq.t())


class NcclBoundary(_Base):
    """cuBLAS GEMM + NCCL all-reduce + eager add and RMSNorm + cuBLAS GEMM (reference ctapp/tp4.py:641-645)."""

    def forward(self, h_r, resid=None):
        y = torch.mm(h_r, self.Wd.t())
        if self.world > 1:
            dist.all_reduce(y)
        return self._post(y, resid)


class NcclFusedNormBoundary(_Base):
    """The stock serving-stack boundary: cuBLAS GEMM + NCCL all-reduce + ONE fused add+RMSNorm kernel + cuBLAS GEMM.
    This is the baseline the pipelined boundary has to beat (the reference's own caveat: its NCCL row carried an
    unfused norm, results/tp4_chain.md:3-11)."""

    def __init__(self, *a):
        super().__init__(*a)
        self.ext = load_tp4()
        n1 = self.Wd.shape[0]
        self.y = torch.empty(self.M, n1, dtype=DTYPE, device=self.dev)
        self.xn = torch.empty(self.M, n1, dtype=DTYPE, device=self.dev)
        self.xo = torch.empty(self.M, n1, dtype=DTYPE, device=self.dev)
        self.out = torch.empty(self.M, self.Wq.shape[0], dtype=DTYPE, device=self.dev)

    def forward(self, h_r, resid=None):
        M = h_r.shape[0]
        torch.mm(h_r, self.Wd.t(), out=self.y[:M])
        if self.world > 1:
            dist.all_reduce(self.y[:M])
        self.ext.add_rmsnorm(self.y[:M], resid, self.gamma, self.xo[:M], self.xn[:M])
        self._x = self.xo[:M]
        return torch.mm(self.xn[:M], self.Wq.t(), out=self.out[:M])


class MultimemBoundary(_Base):
    """cuBLAS GEMM into a symmetric buffer + torch's in-switch (multimem) all-reduce + eager add and norm (reference
    ctapp/tp4.py:573-583).  Needs torch symmetric memory with multicast support."""

    def __init__(self, *a):
        super().__init__(*a)
        import torch.distributed._symmetric_memory as symm_mem
        self.y = symm_mem.empty(self.M, self.Wd.shape[0], dtype=DTYPE, device=self.dev)
        self._h = symm_mem.rendezvous(self.y, self.gn if isinstance(self.gn, str) else dist.group.WORLD.group_name)

    def forward(self, h_r, resid=None):
        torch.mm(h_r, self.Wd.t(), out=self.y)
        torch.ops.symm_mem.multimem_all_reduce_(self.y, "sum", self.gn if isinstance(self.gn, str) else dist.group.WORLD.group_name)
        return self._post(self.y, resid)


class AsyncTpBoundary(_Base):
    """torch's fused matmul + reduce-scatter (the async-TP decomposition), norm on the own rows, all-gather, GEMM (reference
    ctapp/tp4.py:621-638)."""

    def __init__(self, *a):
        super().__init__(*a)
        import torch.distributed._symmetric_memory as symm_mem
        self._gname = self.gn if isinstance(self.gn, str) else dist.group.WORLD.group_name
        symm_mem.enable_symm_mem_for_group(self._gname)
        self.full = torch.empty(self.M, self.Wd.shape[0], dtype=DTYPE, device=self.dev)

    def forward(self, h_r, resid=None):
        from torch.distributed._symmetric_memory import _fused_matmul_reduce_scatter
        m = self.M // self.world
        ys = _fused_matmul_reduce_scatter(h_r, self.Wd.t(), "sum", 0, self._gname)
        if resid is not None:
            ys = ys + resid[self.rank * m:(self.rank + 1) * m]
        self._x = ys                                             # own rows only
        dist.all_gather_into_tensor(self.full, rmsnorm_gamma(ys, self.gamma))
        return torch.mm(self.full, self.Wq.t())


class FlashInferBoundary(_Base):
    """cuBLAS GEMM + FlashInfer's fused all-reduce + residual + RMSNorm kernel (the serving stacks' production path) + cuBLAS
    GEMM (reference ctapp/tp4.py:586-618).  The reduction is not overlapped with the GEMM.  FlashInfer builds its kernels on
    first use."""

    def __init__(self, *a, use_oneshot=None):
        super().__init__(*a)
        from flashinfer.comm import trtllm_create_ipc_workspace_for_all_reduce_fusion as create
        n1 = self.Wd.shape[0]
        self.use_oneshot = use_oneshot
        self.ipc, self.ws = create(self.rank, self.world, self.M, n1, group=dist.group.WORLD)[:2]
        self.y = torch.empty(self.M, n1, dtype=DTYPE, device=self.dev)
        self.resid_out = torch.empty(self.M, n1, dtype=DTYPE, device=self.dev)
        self.norm_out = torch.empty(self.M, n1, dtype=DTYPE, device=self.dev)
        self.zeros = None
        self.gamma_c = self.gamma.contiguous()

    def forward(self, h_r, resid=None):
        from flashinfer.comm import AllReduceFusionPattern, trtllm_allreduce_fusion
        if resid is None:
            if self.zeros is None:
                self.zeros = torch.zeros_like(self.y)
            resid = self.zeros
        torch.mm(h_r, self.Wd.t(), out=self.y)
        trtllm_allreduce_fusion(allreduce_in=self.y, world_size=self.world, world_rank=self.rank, token_num=self.M, hidden_dim=self.y.shape[1],
                                workspace_ptrs=self.ws, launch_with_pdl=False, trigger_completion_at_end=True, fp32_acc=True,
                                pattern_code=AllReduceFusionPattern.kARResidualRMSNorm, use_oneshot=self.use_oneshot, allreduce_out=None,
                                residual_in=resid, residual_out=self.resid_out, norm_out=self.norm_out, quant_out=None, scale_out=None,
                                rms_gamma=self.gamma_c, rms_eps=EPS, scale_factor=None, layout_code=None)
        self._x = self.resid_out
        return torch.mm(self.norm_out, self.Wq.t())

    def destroy(self):
        from flashinfer.comm import trtllm_destroy_ipc_workspace_for_all_reduce_fusion as destroy
        torch.cuda.synchronize(self.dev)
        dist.barrier()
        destroy(self.ipc)


# --------------------------------------------------------------------------- references
@torch.no_grad()
def one_gpu_reference(h_full, Wdown_full, resid, gamma, Wqkv_full, eps=EPS):
    """fp32 chain -> (x_new fp32 (M, n1), out_full fp32 (M, N2)) (reference ctapp/tp4.py:650-656)."""
    x = h_full.float() @ Wdown_full.float().t()
    if resid is not None:
        x = x + resid.float()
    n = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()
    return x, n @ Wqkv_full.float().t()


@torch.no_grad()
def one_gpu_chain_bf16(h_full, Wdown_full, resid, gamma, Wqkv_full):
    """Eager bf16 chain on one GPU (the ideal-timing reference); returns (x, out)."""
    x = torch.mm(h_full, Wdown_full.t())
    if resid is not None:
        x = x + resid
    return x, torch.mm(rmsnorm_gamma(x, gamma), Wqkv_full.t())


def make_inputs(M, dev, seed=1, K=K_FFN, n1=N1):
    """Seeded full-size inputs, generated on the CPU (identical bits for the CPU oracle and every rank): h (M, K) ~ N(0,1),
    resid (M, n1) ~ N(0,1), bf16."""
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(M, K, generator=g).to(DTYPE)
    resid = torch.randn(M, n1, generator=g).to(DTYPE)
    return h.to(dev), resid.to(dev)


def make_weights(dev, seed=0, K=K_FFN, N2_=N2, n1=N1):
    """Seeded full weights, generated on the CPU: Wdown (n1, K) ~ N(0, 1/K), gamma (n1) ~ U(0.5, 1.5), Wqkv (N2_, n1) ~ N(0, 1/n1)."""
    g = torch.Generator().manual_seed(seed)
    Wd = (torch.randn(n1, K, generator=g) * K ** -0.5).to(DTYPE)
    gamma = (0.5 + torch.rand(n1, generator=g)).to(DTYPE)
    Wq = (torch.randn(N2_, n1, generator=g) * n1 ** -0.5).to(DTYPE)
    return Wd.to(dev), gamma.to(dev), Wq.to(dev)


# --------------------------------------------------------------------------- process harness + timing (ctapp/harness.py)
from ctapp import harness as _harness  # noqa: E402
from ctapp.harness import launch, time_one_gpu  # noqa: E402,F401

GLOO = None      # the gloo side group of this process (set by ``launch`` workers, or by the caller)


def barrier():
    dist.barrier(group=GLOO)


def time_step(step, dev, iters, warmup):
    """(per-step median ms with barrier + sync before each call, back-to-back mean ms), both max over ranks
    (reference ctapp/tp4.py:696-723)."""
    return _harness.time_step(step, dev, iters, warmup, GLOO)
