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
FUSIONS = ("none", "pdl", "pdl1", "role", "serial")

# Symmetric buffers of one boundary instance: name -> (shape as a function of the sizes, dtype, wants a multicast address).
# ``t`` = ranks, ``ppo`` = panels per owner, ``tn`` = 256-column tiles of the hidden size, ``P`` = max_M / 128.
_SYMMETRIC = (
    ("inbox", lambda z: (z.t, z.ppo * 128, z.n1), DTYPE, False),        # slot s = partial tiles from source rank s
    ("tile_flags", lambda z: (z.t, z.ppo, z.tn), torch.int32, False),   # [source][owned panel][n-tile], epoch values
    ("panel_flag", lambda z: (z.P,), torch.int32, True),                # epoch values, raised by the owners
    ("rowss", lambda z: (2, z.max_M), torch.float32, True),             # row sums of squares, by epoch parity
    ("xbuf", lambda z: (z.max_M, z.n1), DTYPE, True),                   # new residual stream, even epochs
    ("xbuf1", lambda z: (z.max_M, z.n1), DTYPE, True),                  # ... odd epochs
)


class _Sizes:
    def __init__(self, max_M, n1, world):
        self.max_M, self.n1, self.t = max_M, n1, world
        self.P, self.tn = max_M // 128, n1 // 256
        self.ppo = -(-self.P // world)


class _Buffers:
    """Everything a boundary instance keeps on its GPU: the symmetric buffers of ``_SYMMETRIC`` (tensor + handle each), the
    per-rank scratch, and the address tables the kernels take, derived from the handles."""

    def __init__(self, sizes, dev, group, rank, want_multicast, with_partials=False):
        self.z, self.dev, self.rank = sizes, dev, rank
        self.handles = {}
        table = _SYMMETRIC + ((("partials", lambda z: (z.max_M, z.n1), DTYPE, True),) if with_partials else ())   # in-switch reduction
        for name, shape, dtype, mc in table:
            t, h = _symm(shape(sizes), dtype, dev, group, rank, mc and want_multicast)
            setattr(self, name, t)
            self.handles[name] = h
        self.multicast = want_multicast and all(self.handles[n].multicast_ptr for n, _, _, mc in table if mc)
        z = sizes
        self.rowss_local = torch.zeros(z.max_M, dtype=torch.float32, device=dev)      # owner's accumulators, zeroed per step
        self.panel_done = torch.zeros(z.P, dtype=torch.int32, device=dev)             # arrivals per owned panel
        self.role_ctr = torch.zeros(2, dtype=torch.int32, device=dev)                 # [1] = the shared unit counter (steal)
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status = new_status(dev)
        for t in (self.tile_flags, self.panel_flag, self.rowss):
            t.zero_()

    def peers(self, name, byte_offset=0):
        return [p + byte_offset for p in self.handles[name].buffer_ptrs]

    def mc(self, name, byte_offset=0):
        return self.handles[name].multicast_ptr + byte_offset if self.multicast else 0

    def tables(self):
        """Address tables: where this rank's producer stores at every owner, where its reducer reads and pushes."""
        z, slot = self.z, self.z.ppo * 128 * self.z.n1 * 2
        return dict(
            dst_ptrs=self.peers("inbox", self.rank * slot),                               # my slot in every owner's inbox
            peer_tf=self.peers("tile_flags"),
            inbox_local=[self.inbox.data_ptr() + s * slot for s in range(z.t)],
            peer_x=[self.peers("xbuf"), self.peers("xbuf1")],
            peer_rowss=[self.peers("rowss", par * z.max_M * 4) for par in (0, 1)],
            peer_pf=self.peers("panel_flag"),
            x_mc=[self.mc("xbuf"), self.mc("xbuf1")],
            rowss_mc=[self.mc("rowss", par * z.max_M * 4) for par in (0, 1)],
            pf_mc=self.mc("panel_flag"),
            partials_local=self.partials.data_ptr() if "partials" in self.handles else 0,
            partials_mc=self.mc("partials") if "partials" in self.handles else 0)


class _GraphCache:
    """CUDA graphs of a forward, one per key.  The first call of an instance runs eagerly (capture must not be the first
    thing a context does with these kernels); from then on a key is captured the first time it is seen and replayed."""

    def __init__(self, dev):
        self.dev, self.graphs, self.primed = dev, {}, False

    def run(self, key, enqueue):
        if not self.primed:
            self.primed = True
            enqueue()
            return
        g = self.graphs.get(key)
        if g is None:
            torch.cuda.synchronize(self.dev)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                enqueue()
            self.graphs[key] = g
        g.replay()


def _check_options(world, protocol, fusion, steal, qkv_tile, down_tail, n1, act, cta_pair, N2r, M, max_M):
    if protocol == "v3r" and steal:
        raise ValueError("protocol 'v3r' (in-switch reduction) has no inbox for the consumer's CTAs to read: steal is not available with it")
    if world not in (1, 2, 4, 8):
        raise ValueError(f"world {world} is not supported (1 | 2 | 4 | 8)")
    if protocol not in (True, False, "v3", "v3r", "v5"):
        raise ValueError(f"unknown protocol {protocol!r}")
    if fusion not in FUSIONS:
        raise ValueError(f"fusion {fusion!r} is not available (none | pdl | pdl1 | role | serial)")
    if fusion == "role" and protocol == "v3r":
        raise ValueError("fusion 'role' makes consumer CTAs the reducer; protocol 'v3r' has no inbox for them to read")
    if qkv_tile not in (256, 128):
        raise ValueError(f"qkv_tile {qkv_tile}")
    if not (down_tail == "auto" or (isinstance(down_tail, int) and 0 <= down_tail <= n1 // 256)):
        raise ValueError(f"down_tail {down_tail!r}")
    if M % 128 or n1 % 256 or max_M % 128 or M > max_M:
        raise ValueError(f"M={M} / max_M={max_M} must be multiples of 128 with M <= max_M, n1={n1} a multiple of 256")
    if act and not (cta_pair and qkv_tile == 256 and N2r % 256 == 0):
        raise ValueError("act needs the CTA-pair consumer and N2r % 256 == 0")


class CtappBoundary:
    """CTA-pipelined boundary, panel-ownership protocol with unicast value flags (the reference's protocol "v5",
    ctapp/tp4.py:60-504), for world in {1, 2, 4, 8}.

    Per forward: ``tp4_step`` (epoch += 1, zero the per-step accumulators) -> producer GEMM mode 7 on ``SMs - R`` SMs ||
    owner reducer (``red_blocks`` CTAs of ``red_threads`` threads) -> consumer GEMM mode 5 / 8 on ``SMs - R`` SMs.  All flags
    are epoch values, so one instance sized ``max_M`` serves every M <= max_M with M % 128 == 0; ``out`` and ``x()`` are
    views of the first M rows.

    protocol: "v5" (default here) = unicast pushes; True / "v3" = NVLS variant: the same panel-ownership protocol, but the owner
    reducer pushes x, the row sums and the panel flags with ``multimem.st`` on multicast addresses, so each row leaves the
    owner once and the NVSwitch replicates it (needs one process per GPU, >= 2 ranks, torch symmetric memory with multicast;
    falls back to unicast with a warning otherwise).  "v3r" = "v3" plus the in-switch reduction of the reference's v3 reducer
    (csrc/ctapp_tp4.cuh:458-536): every producer keeps its partial tiles in its own memory and only raises the owner's tile
    flag; the owner reads each 16 bytes of the cross-rank sum with one ``multimem.ld_reduce`` (fp32 accumulation inside the
    switch) instead of ``world`` loads from its inbox.  Same flags and order as v5.  Opt-in, because of its numerics: the
    switch returns the partials' sum as bf16 and the residual is added after that rounding, one bf16 rounding more than v5; x
    stays within the bounds (max 2e-2, mean 1e-3 of the RMS) but ``out`` was measured at a mean error of 1.9e-3 of its RMS
    against v5's rounding model (max 1.5e-2).  Fastest variant at TP4, slower than v5 at TP2.  False = the two GEMMs alone (no exchange, no residual): the floor the
    protocol is measured against.
    fusion: "none" = reducer on a side stream, consumer after the producer in stream order;
            "pdl"  = as "none" and the consumer is launched as the producer's programmatic dependent, so its CTAs start
                     as producer CTAs retire (the per-panel flags carry the data dependency);
            "pdl1" = one stream: reducer (raises the launch trigger at entry) -> producer -> consumer, each the programmatic
                     dependent of the one before (reference ctapp/tp4.py:316-320);
            "role" = two launches on one stream, no reducer kernel: the producer GEMM on ``SMs - R`` SMs raises the launch
                     trigger, the consumer GEMM (mode 8, every SM) is its programmatic dependent, and the first R of its CTAs
                     to arrive -- those that land on the SMs the producer leaves free -- run the owner reducer's static
                     shares before they take GEMM tiles (reference ctapp/tp4.py:312-315, csrc/ctapp_tp4.cuh:913-925); with
                     ``steal`` every consumer CTA claims units from the shared counter instead;
            "serial" = step, producer, reducer, consumer on one stream, nothing concurrent on this GPU (used where a
                     single GPU plays every rank).
    steal: the consumer runs in mode 8: each of its CTAs first claims owner-reducer units from the counter the dedicated
    reducer CTAs claim from, as long as there are units whose tiles have arrived and that no reducer warp has taken yet, so CTAs
    that become resident as the producer's retire drain what the reducer has fallen behind by, and start their own tiles at
    once when the reducer keeps pace
    (reference ctapp/tp4.py:110-114, csrc/ctapp_tp4.cuh:913-925).  ``R=0`` with steal leaves the reduction to them alone
    (with fusion "serial" that only works for world 1: a consumer that reduces its own panels and then waits for the other
    ranks' panels needs those ranks' consumers to run at the same time).
    use_graph: forwards are captured into CUDA graphs keyed by (parity, M); inputs are copied into static buffers
    before each replay (``graph_bind`` captures the caller's tensors instead).
    act: the consumer's weight is a gate/up projection with rows interleaved by ``interleave_gate_up``; its epilogue applies
    silu(gate) * up and ``out`` is (M, N2r / 2): the activation costs no pass over memory of its own.
    cta_pair: both GEMMs run as CTA pairs (``cta_group::2``, 256-row tiles; the protocol's unit stays the 128-row panel);
    the producer then works on 256 x 512 tiles (raising two tile flags per tile) up to TP2 when M is large enough to give
    every pair such a tile, on 256 x 256 tiles otherwise; "wide" / "narrow" force either; False = one CTA per 128-row tile.
    ``group_name``: a torch.distributed group name (one process per GPU) or a ``ctapp.symm.LocalGroup`` (one process
    drives every rank's GPU).
    """

    def __init__(self, M, Kr, N2r, rank, world, group_name, device, resid=True, protocol="v5", use_graph=False, R=None,
                 qkv_raster=2, qkv_swizzle=1, max_M=None, down_raster=None, red_threads=1024, red_blocks=None, red_variant=1,
                 fusion="none", qkv_tile=256, role_rows=4, down_swizzle=1, pdl_trigger=None, trace=None, role_stages=0, steal=False,
                 down_tail="auto", graph_bind=False, n1=N1, eps=EPS, cta_pair=True, act=False):
        max_M = max_M or M
        _check_options(world, protocol, fusion, steal, qkv_tile, down_tail, n1, act, cta_pair, N2r, M, max_M)
        self.ext = load_tp4()
        self.dev = device if isinstance(device, torch.device) else torch.device("cuda", device)
        self.M, self.max_M, self.Kr, self.N2r, self.rank, self.world, self.group = M, max_M, Kr, N2r, rank, world, group_name
        self.n1, self.eps, self.cta_pair, self.act = n1, eps, int(bool(cta_pair)), int(bool(act))
        # producer tile: CTA pairs work on 256 x 512 tiles (a quarter less operand traffic; TP2, M=4096: 0.921 against 0.938 ms
        # for the whole boundary) whenever that still gives every pair a tile; "wide" / "narrow" force the choice
        self._down_wide = {"wide": True, "narrow": False}.get(cta_pair) if isinstance(cta_pair, str) else (None if cta_pair else False)
        self.use_resid, self.protocol, self.v5 = resid, bool(protocol), bool(protocol)
        self.use_graph, self.graph_bind = use_graph, bool(graph_bind)
        self.fusion, self.steal = fusion, bool(steal)
        # SM split: R SMs are left to the owner reducer.  Measured on B200 at M=4096: TP2 best with 4; TP4 0.515 / 0.509 / 0.525 ms
        # with 8 / 12 / 16; TP8 0.519 / 0.378 ms with 4 / 8 (a reducer SM moves about 80 GB/s whatever it runs, and at TP8 the
        # two GEMMs are over before 8 such SMs are through); with a TP8 rank's GEMM shapes on 4 GPUs 0.347 / 0.311 / 0.307 / 0.312 ms
        # with 8 / 12 / 16 / 24
        self.nsm = torch.cuda.get_device_properties(self.dev).multi_processor_count
        self.R = (4 if world <= 2 else 8 if world <= 4 else 12) if R is None else int(R)
        # R = 0 gives both GEMMs every SM.  The reduction is then done by ``red_blocks`` small reducer CTAs that share SMs with
        # the GEMMs' CTAs (a GEMM CTA leaves more than half of an SM's registers and nearly all its thread slots free; choose
        # ``red_threads`` <= 512 so that both fit), by the consumer's CTAs (``steal``), or by both
        if fusion == "role" and self.R == 0 and not self.steal:
            raise ValueError("fusion 'role' needs R > 0 (that many consumer CTAs become the reducer) or steal=True")
        if self.R == 0 and not self.steal and not red_blocks:
            raise ValueError("R=0 (no SMs set aside for the reducer) needs red_blocks (reducer CTAs sharing SMs with the GEMMs) or steal=True")
        self.sms = self.qkv_sms = self.nsm - self.R
        self.red_threads, self.red_blocks = red_threads, self.R if red_blocks is None else int(red_blocks)
        if fusion == "role":          # no reducer kernel: the consumer takes every SM, its first CTAs land on the R the producer leaves
            self.qkv_sms, self.red_blocks = self.nsm, 0
        # tile orders of the three kernels
        self.qkv_raster, self.qkv_swizzle, self.qkv_tile = qkv_raster, qkv_swizzle, qkv_tile
        self.down_raster, self.down_swizzle, self.down_tail = down_raster or 1, down_swizzle, down_tail
        self.pdl_trigger = int(fusion in ("pdl", "pdl1", "role")) if pdl_trigger is None else int(pdl_trigger)
        self.trace = bool(int(os.environ.get("CTAPP_TRACE", "0"))) if trace is None else bool(trace)
        want_mc = protocol in (True, "v3", "v3r") and world >= 2 and not isinstance(group_name, LocalGroup)
        if protocol in (True, "v3", "v3r") and not want_mc:
            log.warning("ctapp: NVLS needs one process per GPU and at least 2 ranks; using unicast pushes")
        sizes = _Sizes(max_M, n1, world)
        with torch.cuda.device(self.dev):
            self.ext.preload(self.dev.index)
            self.buf = _Buffers(sizes, self.dev, group_name, rank, want_mc, with_partials=want_mc and protocol == "v3r")
            if want_mc and not self.buf.multicast:
                log.warning("ctapp: no multicast address on this system; using unicast pushes")
            self.nvls = self.buf.multicast
            self.ldreduce = self.nvls and protocol == "v3r"       # the switch sums the partials; producers store locally
            self.tab = self.buf.tables()
            self.trace_down = torch.zeros(self.nsm * 8, dtype=torch.int64, device=self.dev)
            self.trace_qkv = torch.zeros(self.nsm * 8, dtype=torch.int64, device=self.dev)
            self.trace_red = torch.zeros(sizes.P, dtype=torch.int64, device=self.dev)
            self.side = torch.cuda.Stream(device=self.dev)
            self.fork, self.join = torch.cuda.Event(), torch.cuda.Event()
            self._out_full = torch.empty(max_M, N2r // 2 if self.act else N2r, dtype=DTYPE, device=self.dev)
            self._floor_y = None
            static = use_graph and not self.graph_bind
            self.h_static = torch.empty(max_M, Kr, dtype=DTYPE, device=self.dev) if static else None
            self.resid_static = torch.empty(max_M, n1, dtype=DTYPE, device=self.dev) if static and resid else None
            torch.cuda.synchronize(self.dev)
        _group_barrier(group_name)
        self.ppo = sizes.ppo
        self.out = self._out_full[:M]
        self.epoch = 0
        self._last = (0, M)          # (parity, M) of the most recent forward
        self.Wd = self.Wq = None
        self._graphs = _GraphCache(self.dev)
        self._enqueue = {"serial": self._enqueue_serial, "none": self._enqueue_forked, "pdl": self._enqueue_forked,
                         "pdl1": self._enqueue_chained, "role": self._enqueue_role}[fusion]

    # the buffers tests and benches look at, by their reference names
    inbox = property(lambda self: self.buf.inbox)
    tile_flags = property(lambda self: self.buf.tile_flags)
    panel_flag = property(lambda self: self.buf.panel_flag)
    rowss = property(lambda self: self.buf.rowss)
    xbuf = property(lambda self: self.buf.xbuf)
    xbuf1 = property(lambda self: self.buf.xbuf1)
    xbufs = property(lambda self: (self.buf.xbuf, self.buf.xbuf1))
    rowss_local = property(lambda self: self.buf.rowss_local)
    panel_done = property(lambda self: self.buf.panel_done)
    role_ctr = property(lambda self: self.buf.role_ctr)
    epoch_dev = property(lambda self: self.buf.epoch_dev)
    status = property(lambda self: self.buf.status)

    # ---- the three kernels of a step
    def tail_cols(self, M):
        """n-tiles the producer leaves for its panel-major tail (reference ctapp/tp4.py:262-267)."""
        if self.down_tail != "auto":
            return self.down_tail
        if (self.down_raster, self.down_swizzle) != (1, 1):
            return 0
        return min(16 if M >= 2048 else 8, self.n1 // 256)

    def down_pair(self, M):
        """``cta_pair`` value of the producer launch for M rows: 0 one CTA per tile, 1 CTA pairs on 256 x 256, 2 on 256 x 512."""
        if not self.cta_pair or self.n1 % 512:
            return self.cta_pair
        wide = self._down_wide
        if wide is None:      # measured at M=4096: TP2 (K=14336 per rank) gains 1.5-2 % on the whole boundary, TP4 (K=7168) loses 2 %:
            wide = self.world <= 2 and (M // 256) * (self.n1 // 512) >= self.sms // 2      # coarser tiles reach the reducer later
        return 2 if wide else 1

    def _stamps(self, t):
        return t.data_ptr() if self.trace else 0

    def _reducer_kwargs(self, M, resid, parity):
        """What the owner reducer needs, under the names both ``tp4_reduce`` and the mode-8 ``tp4_qkv`` take."""
        t = self.tab
        return dict(resid=resid, inbox_ptrs=t["inbox_local"], peer_x=t["peer_x"][parity], peer_rowss=t["peer_rowss"][parity],
                    peer_panel_flag=t["peer_pf"], rowss_local=self.buf.rowss_local, panel_done=self.buf.panel_done,
                    panels_per_owner=self.ppo, x_mc_ptr=t["x_mc"][parity], rowss_mc_ptr=t["rowss_mc"][parity],
                    panel_flag_mc_ptr=t["pf_mc"], red_trace=self._stamps(self.trace_red), status=self.buf.status)

    def launch_reducer(self, M, resid, parity, unit_log=None):
        if self.red_blocks == 0:
            return
        self.ext.tp4_reduce(M, self.rank, self.world, 0, self.down_raster, self.red_blocks, self.buf.tile_flags, version=5,
                            epoch_dev=self.buf.epoch_dev, threads=self.red_threads, swz=self.down_swizzle, n1=self.n1,
                            unit_ctr=self.buf.role_ctr[1:] if self.steal else 0, tail_cols=self.tail_cols(M),
                            pdl_trigger=int(self.fusion == "pdl1"), unit_log=unit_log,
                            partials_mc_ptr=self.tab["partials_mc"] if self.ldreduce else 0, **self._reducer_kwargs(M, resid, parity))

    def launch_producer(self, h_r, Wd, M, tile_log=None, sms=None):
        t = self.tab
        if self.ldreduce:      # every "destination" is this rank's own partial buffer, rows in place: only the flags travel
            dst = dict(dst_ptrs=[t["partials_local"]] * self.world, dst_rows=self.max_M, dst_global=1)
        else:
            dst = dict(dst_ptrs=t["dst_ptrs"], dst_rows=self.ppo * 128)
        self.ext.tp4_down(h_r, Wd, None, self.down_raster, self.down_swizzle, 7, self.rank, self.world, 0, sms=self.sms if sms is None else sms,
                          epoch_dev=self.buf.epoch_dev, peer_tile_flags=t["peer_tf"], **dst,
                          panels_per_owner=self.ppo, pdl_trigger=self.pdl_trigger, pdl=int(self.fusion == "pdl1"),
                          trace=self._stamps(self.trace_down), tail_cols=self.tail_cols(M), status=self.buf.status, cta_pair=self.down_pair(M),
                          tile_log=tile_log)

    def launch_consumer(self, Wq, M, parity, resid=None):
        common = dict(sms=self.qkv_sms, pdl=int(self.fusion in ("pdl", "pdl1", "role")), epoch_dev=self.buf.epoch_dev, tile=self.qkv_tile,
                      trace=self._stamps(self.trace_qkv), eps=self.eps, cta_pair=self.cta_pair, act=self.act)
        args = (self.xbufs[parity][:M], Wq, self._out_full[:M], self.qkv_raster, self.qkv_swizzle)
        role = self.fusion == "role"
        if not self.steal and not role:
            self.ext.tp4_qkv(*args, 5, 0, self.buf.panel_flag, 1, self.buf.rowss[parity], status=self.buf.status, **common)
            return
        self.ext.tp4_qkv(*args, 8, 0, self.buf.panel_flag, 1, self.buf.rowss[parity], role_ctr=self.buf.role_ctr, rank=self.rank,
                         world=self.world, red_order=2 if self.down_raster == 2 else 1, red_swz=self.down_swizzle,
                         tile_flags=self.buf.tile_flags, red_tail=self.tail_cols(M), help_all=int(self.red_blocks == 0),
                         R=self.R if role else 0, red_dyn=int(self.steal), **self._reducer_kwargs(M, resid, parity), **common)

    # ---- how the kernels of one step are put on streams
    def _step(self, M):
        self.ext.tp4_step(self.buf.epoch_dev, self.buf.rowss_local, self.buf.panel_done, M, self.buf.role_ctr)

    def _enqueue_serial(self, h_r, resid, parity, Wd, Wq, M):
        self._step(M)
        self.launch_producer(h_r, Wd, M)
        self.launch_reducer(M, resid, parity)
        self.launch_consumer(Wq, M, parity, resid)

    def _enqueue_forked(self, h_r, resid, parity, Wd, Wq, M):
        """Reducer on the side stream, forked after the step kernel and joined after the consumer."""
        main = torch.cuda.current_stream(self.dev)
        self._step(M)
        self.fork.record(main)
        self.side.wait_event(self.fork)
        with torch.cuda.stream(self.side):
            self.launch_reducer(M, resid, parity)
            self.join.record(self.side)
        self.launch_producer(h_r, Wd, M)
        self.launch_consumer(Wq, M, parity, resid)
        main.wait_event(self.join)

    def _enqueue_chained(self, h_r, resid, parity, Wd, Wq, M):
        """One stream, three programmatic launches: the reducer lets the producer in at once, the producer the consumer."""
        self._step(M)
        self.launch_reducer(M, resid, parity)
        self.launch_producer(h_r, Wd, M)
        self.launch_consumer(Wq, M, parity, resid)

    def _enqueue_role(self, h_r, resid, parity, Wd, Wq, M):
        """One stream, two launches: the producer lets the consumer in at once; consumer CTAs are the reducer."""
        self._step(M)
        self.launch_producer(h_r, Wd, M)
        self.launch_consumer(Wq, M, parity, resid)

    def _enqueue_floor(self, h_r, Wd, Wq, M):
        """The two GEMMs with the same SM split and tile orders, no exchange (reference ctapp/tp4.py:365-369)."""
        if self._floor_y is None:
            self._floor_y = torch.empty(self.max_M, self.n1, dtype=DTYPE, device=self.dev)
        self.ext.tp4_down(h_r, Wd, self._floor_y[:M], self.down_raster, self.down_swizzle, 0, self.rank, self.world, 0, sms=self.sms,
                          tail_cols=self.tail_cols(M), cta_pair=self.down_pair(M))
        self.ext.tp4_qkv(self._floor_y[:M], Wq, self._out_full[:M], self.qkv_raster, self.qkv_swizzle, 0, 0, sms=self.qkv_sms, tile=self.qkv_tile,
                         cta_pair=self.cta_pair, act=self.act)

    # ---- public API
    def warmup(self):
        """Kept for API compatibility: every kernel is loaded at construction (``ctapp_preload``), so nothing is launched."""

    def _weights(self, Wd, Wq):
        Wd = self.Wd if Wd is None else Wd
        Wq = self.Wq if Wq is None else Wq
        if Wd is None or Wq is None:
            raise ValueError("no weights: call set_weights() or pass Wd / Wq")
        for w, shape, name in ((Wd, (self.n1, self.Kr), "Wd"), (Wq, (self.N2r, self.n1), "Wq")):
            if tuple(w.shape) != shape or w.dtype != DTYPE or not w.is_contiguous():
                raise ValueError(f"{name} must be a contiguous bf16 {shape} tensor, got {tuple(w.shape)} {w.dtype}")
        return Wd, Wq

    def set_weights(self, Wdown_r, Wqkv_r_folded):
        """Default weights (used when forward() gets none; baked into the graphs when use_graph)."""
        self.Wd, self.Wq = self._weights(Wdown_r, Wqkv_r_folded)

    def _inputs(self, h_r, resid):
        M = h_r.shape[0]
        if M % 128 or not 0 < M <= self.max_M:
            raise ValueError(f"M={M} must be a positive multiple of 128 up to max_M={self.max_M}")
        for t, shape, name in ((h_r, (M, self.Kr), "h_r"), (resid, (M, self.n1), "resid")):
            if t is not None and (tuple(t.shape) != shape or t.dtype != DTYPE or not t.is_contiguous()):
                raise ValueError(f"{name} must be a contiguous bf16 {shape} tensor, got {tuple(t.shape)} {t.dtype}")
        return M

    def forward(self, h_r, resid=None, Wd=None, Wq=None):
        """Wd (n1, Kr) / Wq (N2r, n1, gamma folded): bf16 contiguous weights for this call (no copy; they must stay alive
        until the stream work finishes); default = those from set_weights.  Per-call weights are not supported with use_graph."""
        if self.use_graph and not (Wd is None and Wq is None):
            raise ValueError("per-call weights are not supported with use_graph")
        Wd, Wq = self._weights(Wd, Wq)
        resid = resid if self.use_resid else None
        M = self._inputs(h_r, resid)
        self.out = self._out_full[:M]
        with torch.cuda.device(self.dev):
            if not self.protocol:
                self._last = (0, M)
                self._enqueue_floor(h_r, Wd, Wq, M)
                return self.out
            self.epoch += 1
            parity = self.epoch & 1
            self._last = (parity, M)
            if resid is not None and resid.data_ptr() == self.xbufs[parity].data_ptr():
                raise ValueError("resid aliases the x buffer this forward writes")
            if not self.use_graph:
                self._enqueue(h_r, resid, parity, Wd, Wq, M)
                return self.out
            key = (parity, M)
            if self.graph_bind:
                key += (h_r.data_ptr(), resid.data_ptr() if resid is not None else 0)
            else:
                self.h_static[:M].copy_(h_r)
                h_r = self.h_static[:M]
                if resid is not None:
                    self.resid_static[:M].copy_(resid)
                    resid = self.resid_static[:M]
            self._graphs.run(key, lambda: self._enqueue(h_r, resid, parity, Wd, Wq, M))
            return self.out

    def x(self):
        """New residual (M, n1) of the most recent forward; valid until two forwards later (x is double-buffered)."""
        parity, M = self._last
        return self._floor_y[:M] if not self.protocol else self.xbufs[parity][:M]

    def check(self):
        """Synchronise this rank's device and raise if a device-side wait gave up."""
        torch.cuda.synchronize(self.dev)
        check_status(self.buf.status, f"boundary rank {self.rank}")

    def trace_summary(self):
        """CTAPP_TRACE stamps of the most recent eager forward, in us relative to the first producer CTA's entry."""
        torch.cuda.synchronize(self.dev)
        prod, cons = (t.view(-1, 8).cpu() for t in (self.trace_down, self.trace_qkv))
        prod, cons = prod[prod[:, 0] > 0], cons[cons[:, 0] > 0]
        if prod.shape[0] == 0:
            return {}
        origin = int(prod[:, 0].min())
        rel_us = lambda v: (int(v) - origin) / 1e3  # noqa: E731
        out = {"prod_ctas": int(prod.shape[0]), "prod_entry_max": rel_us(prod[:, 0].max()), "prod_first_tile_max": rel_us(prod[:, 1].max()),
               "prod_end_min": rel_us(prod[:, 7].min()), "prod_end_max": rel_us(prod[:, 7].max()), "cons_ctas": int(cons.shape[0])}
        owned = torch.arange(self.rank, self._last[1] // 128, self.world)
        pub = self.trace_red.cpu()[owned]
        if pub.numel() and int(pub.min()) > 0:
            out["red_first_panel"], out["red_last_panel"] = rel_us(pub.min()), rel_us(pub.max())
        if cons.shape[0]:
            out.update(cons_entry_min=rel_us(cons[:, 0].min()), cons_first_tile_min=rel_us(cons[:, 1].min()), cons_end_max=rel_us(cons[:, 7].max()))
        return out


def forward_lockstep(bds, h_rs, resids, Wds, Wqs):
    """One forward of every rank of a ``LocalGroup`` from this process, phase by phase: all producers, then all owner
    reducers, then all consumers.  When several ranks share a GPU (one device playing all ranks) no kernel is ever
    launched before the kernels it waits for, so nothing waits on the device; with one GPU per rank the phases of different
    ranks still overlap across GPUs.  Returns the list of per-rank outputs."""
    Ms = [h.shape[0] for h in h_rs]
    for bd, M in zip(bds, Ms):
        bd.epoch += 1
        bd._last = (bd.epoch & 1, M)
        bd.out = bd._out_full[:M]
        with torch.cuda.device(bd.dev):
            bd._step(M)
    for bd, h, Wd, M in zip(bds, h_rs, Wds, Ms):
        with torch.cuda.device(bd.dev):
            bd.launch_producer(h, Wd, M)
    for bd, r, M in zip(bds, resids, Ms):
        with torch.cuda.device(bd.dev):
            bd.launch_reducer(M, r if bd.use_resid else None, bd._last[0])
    for bd, Wq, r, M in zip(bds, Wqs, resids, Ms):
        with torch.cuda.device(bd.dev):
            bd.launch_consumer(Wq, M, bd._last[0], r if bd.use_resid else None)
    return [bd.out for bd in bds]


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
    ``get`` at the same point.  Same constructor as reference ctapp/tp4.py:507-554; ``max_instances`` is accepted for that
    reason (one instance serves every M here whatever the protocol).
    """

    def __init__(self, Kr, N2r, rank, world, group_name, device, R=None, min_M=512, max_instances=4,
                 qkv_raster=2, qkv_swizzle=1, protocol="v5", max_M=8192, **v5kw):
        if protocol not in ("v3", "v3r", "v5"):
            raise ValueError(f"unknown protocol {protocol!r}")
        self.min_M, self.max_M, self.max_instances, self.protocol = min_M, max_M, max_instances, protocol
        self._where = (Kr, N2r, rank, world, group_name, device)
        self._options = dict(R=R, qkv_raster=qkv_raster, qkv_swizzle=qkv_swizzle, protocol=protocol, max_M=max_M, **v5kw)
        self._inst = {}       # max_M -> instance (at most one entry)

    def supports(self, M):
        return M % 128 == 0 and self.min_M <= M <= self.max_M

    def get(self, M):
        if not self.supports(M):
            return None
        if self.max_M not in self._inst:
            self._inst[self.max_M] = CtappBoundary(self.max_M, *self._where, **self._options)
        return self._inst[self.max_M]


# --------------------------------------------------------------------------- comparison boundaries
class _StockBoundary:
    """What the pipelined boundary is compared with: down-projection, some all-reduce, add + RMSNorm, next projection, each a
    separate step.  Subclasses say how the partial sums are reduced (``reduced``) and how the norm is applied (``normed``);
    ``forward(h_r, resid)`` and ``x()`` are the pipelined boundary's."""

    def __init__(self, M, rank, world, group_name, device, Wdown_r, Wqkv_r, gamma):
        self.M, self.rank, self.world, self.gn, self.dev = M, rank, world, group_name, device
        self.w_down, self.w_next, self.gamma = Wdown_r, Wqkv_r, gamma.to(DTYPE)
        self.residual = None

    def x(self):
        return self.residual

    def partial(self, h_r):
        return torch.mm(h_r, self.w_down.t())

    def reduced(self, y):
        return y

    def normed(self, y, resid):
        """(new residual, normalised activations)"""
        x = y if resid is None else y + resid
        return x, rmsnorm_gamma(x, self.gamma)

    def forward(self, h_r, resid=None):
        self.residual, n = self.normed(self.reduced(self.partial(h_r)), resid)
        return torch.mm(n, self.w_next.t())


class NcclBoundary(_StockBoundary):
    """cuBLAS GEMM + NCCL all-reduce + eager add and RMSNorm + cuBLAS GEMM (reference ctapp/tp4.py:641-645)."""

    def reduced(self, y):
        if self.world > 1:
            dist.all_reduce(y)
        return y


class NcclFusedNormBoundary(NcclBoundary):
    """The stock serving-stack boundary: cuBLAS GEMM + NCCL all-reduce + ONE fused add+RMSNorm kernel + cuBLAS GEMM.
    This is the baseline the pipelined boundary has to beat (the reference's own caveat: its NCCL row carried an
    unfused norm, results/tp4_chain.md:3-11).  Works in preallocated buffers."""

    def __init__(self, *a):
        super().__init__(*a)
        self.ext = load_tp4()
        n1 = self.w_down.shape[0]
        new = lambda cols: torch.empty(self.M, cols, dtype=DTYPE, device=self.dev)  # noqa: E731
        self.y, self.xn, self.xo, self.out = new(n1), new(n1), new(n1), new(self.w_next.shape[0])

    def partial(self, h_r):
        return torch.mm(h_r, self.w_down.t(), out=self.y[:h_r.shape[0]])

    def normed(self, y, resid):
        rows = y.shape[0]
        self.ext.add_rmsnorm(y, resid, self.gamma, self.xo[:rows], self.xn[:rows])
        return self.xo[:rows], self.xn[:rows]

    def forward(self, h_r, resid=None):
        self.residual, n = self.normed(self.reduced(self.partial(h_r)), resid)
        return torch.mm(n, self.w_next.t(), out=self.out[:n.shape[0]])


class MultimemBoundary(_StockBoundary):
    """cuBLAS GEMM into a symmetric buffer + torch's in-switch (multimem) all-reduce + eager add and norm (reference
    ctapp/tp4.py:573-583).  Needs torch symmetric memory with multicast support."""

    def __init__(self, *a):
        super().__init__(*a)
        import torch.distributed._symmetric_memory as sm
        self._group = self.gn if isinstance(self.gn, str) else dist.group.WORLD.group_name
        self.y = sm.empty(self.M, self.w_down.shape[0], dtype=DTYPE, device=self.dev)
        self._handle = sm.rendezvous(self.y, self._group)

    def partial(self, h_r):
        return torch.mm(h_r, self.w_down.t(), out=self.y)

    def reduced(self, y):
        torch.ops.symm_mem.multimem_all_reduce_(y, "sum", self._group)
        return y


class AsyncTpBoundary(_StockBoundary):
    """torch's fused matmul + reduce-scatter (the async-TP decomposition), norm on the own rows, all-gather, GEMM (reference
    ctapp/tp4.py:621-638)."""

    def __init__(self, *a):
        super().__init__(*a)
        import torch.distributed._symmetric_memory as sm
        self._group = self.gn if isinstance(self.gn, str) else dist.group.WORLD.group_name
        sm.enable_symm_mem_for_group(self._group)
        self.gathered = torch.empty(self.M, self.w_down.shape[0], dtype=DTYPE, device=self.dev)

    def forward(self, h_r, resid=None):
        from torch.distributed._symmetric_memory import _fused_matmul_reduce_scatter as matmul_rs
        rows = self.M // self.world
        mine = matmul_rs(h_r, self.w_down.t(), "sum", 0, self._group)
        if resid is not None:
            mine = mine + resid[self.rank * rows:(self.rank + 1) * rows]
        self.residual = mine                                      # own rows only
        dist.all_gather_into_tensor(self.gathered, rmsnorm_gamma(mine, self.gamma))
        return torch.mm(self.gathered, self.w_next.t())


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
