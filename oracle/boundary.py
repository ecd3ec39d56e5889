"""Oracle for the tensor-parallel layer boundary (TEST INFRASTRUCTURE, never on a product path).

down-proj partial GEMM -> cross-rank sum + residual -> RMSNorm (gamma folded into the next weight)
-> next projection.  Restates for the CPU:
  * the fp32 reference chain                          (reference ctapp/tp4.py:650-656)
  * weight sharding and gamma folding                 (reference ctapp/tp4.py:38-56)
  * the producer tile order "m-fast head, panel-major tail"   (reference csrc/ctapp_tp4.cuh:897-906)
  * the owner reducer's unit order                    (reference csrc/ctapp_tp4.cuh:551-565)
  * panel ownership / inbox / flag indexing           (reference csrc/ctapp_tp4.cuh:279-280,612-614,658-663;
                                                       ctapp/tp4.py:197,262-267)
  * the rounding model of the device path             (reference csrc/ctapp_tp4.cuh:589-598,676-679;
                                                       csrc/gemm_tp4.cu:26-39)
The reference hard-codes 4 ranks; everything here takes ``world``.
"""
from __future__ import annotations

import numpy as np

EPS = 1e-5
N1 = 8192       # hidden size: down-proj N and RMSNorm width
K_FFN = 28672
N2 = 10240      # fused QKV width
PANEL = 128     # rows per panel
UNIT_COLS = 256  # columns per reducer unit == producer tile width
QUARTERS = 4    # a unit covers a 32-row quarter of a panel


# ------------------------------------------------------------------------------------------ integers
def panels_per_owner(max_M, world):
    """Rows of inbox per source slot, in panels: ceil(max_M / 128 / world)   (ctapp/tp4.py:197)."""
    return -(-(max_M // PANEL) // world)


def panels_owned(M, rank, world):
    """Number of 128-row panels m < M/128 with m % world == rank   (csrc/ctapp_tp4.cuh:612-614)."""
    P = M // PANEL
    return (P - 1 - rank) // world + 1 if P > rank else 0


def tail_cols(M, raster=1, swizzle=1, tiles_n=N1 // UNIT_COLS):
    """Default width (in n-tiles) of the panel-major tail of the producer order   (ctapp/tp4.py:262-267)."""
    if raster != 1 or swizzle != 1:
        return 0
    return min(16 if M // PANEL >= 16 else 8, tiles_n)


def remap_tile(L, TM, TN, C):
    """Linear producer tile index L -> (m, n).  The first TM*(TN-C) indices walk n-tiles 0..TN-C-1 with m
    fastest; the rest walk the last C n-tiles panel by panel (n fastest)   (csrc/ctapp_tp4.cuh:897-906).
    C == 0 is plain m-fastest order."""
    head = TM * (TN - C)
    if L < head:
        return L % TM, L // TM
    L2 = L - head
    return L2 // C, TN - C + L2 % C


def unit_map(u, Pr, tiles_n, tail, order=1, swz=1):
    """Reducer unit u -> (owned panel j, n-tile, quarter q), following the producer order restricted to
    this rank's panels   (csrc/ctapp_tp4.cuh:551-565): the tail order when tail > 0; otherwise order 1 = m fastest
    (n-major; with swz > 1 in groups of swz n-tiles: for each group, for each owned panel, the group's n-tiles),
    order 2 = panel by panel."""
    q, t = u % QUARTERS, u // QUARTERS
    if tail > 0:
        head = Pr * (tiles_n - tail)
        if t < head:
            return t % Pr, t // Pr, q
        t2 = t - head
        return t2 // tail, tiles_n - tail + t2 % tail, q
    if order == 2:
        return t // tiles_n, t % tiles_n, q
    if swz <= 1:
        return t % Pr, t // Pr, q
    g = t // swz
    return g % Pr, (g // Pr) * swz + t % swz, q


def tile_order(order, TM, TN, group_rows=1, tail=0):
    """(m, n) of every schedule position of a GEMM with TM x TN tiles, for the three static orders of the kernels: 0 = groups of
    ``group_rows`` tile rows, n-major inside a group (the last group may be short); 1 = ``remap_tile`` with ``tail`` columns;
    2 = n fastest.  Order 1 restates csrc/ctapp_tp4.cuh:897-906; order 0 is the chain's grouped producer order
    (ctapp/pipeline.py:48-51) as a position -> tile function; order 2 is row-major."""
    out = []
    for L in range(TM * TN):
        if order == 2:
            out.append((L // TN, L % TN))
        elif order == 1:
            out.append(remap_tile(L, TM, TN, tail))
        else:
            g = max(group_rows, 1)
            grp, r = divmod(L, g * TN)
            m0 = grp * g
            rows = min(g, TM - m0)
            out.append((m0 + r % rows, r // rows))
    return out


def tile_flag_index(src, j, n, ppo, tiles_n=N1 // UNIT_COLS):
    """Index into an owner's tile_flags[world][ppo][tiles_n] for source rank src, owned panel j, n-tile n."""
    return (src * ppo + j) * tiles_n + n


def owner_of(m, world):
    """(owner rank, owned-panel index j) of global panel m."""
    return m % world, m // world


class BoundarySim:
    """Sequential model of one boundary step on ``world`` ranks: which flags / counters every rank holds
    after a step with epoch ``e``.  Used to pin the protocol state the device path must leave behind
    (reference tests/test_tp4.py:202-213: every tile flag of the owned panels and every panel flag == epoch)."""

    def __init__(self, max_M, world, tiles_n=N1 // UNIT_COLS):
        self.world, self.tiles_n = world, tiles_n
        self.ppo = panels_per_owner(max_M, world)
        self.tile_flags = np.zeros((world, world, self.ppo, tiles_n), dtype=np.int64)   # [owner][src][j][n]
        self.panel_flag = np.zeros((world, max_M // PANEL), dtype=np.int64)             # [rank][m]
        self.panel_done = np.zeros((world, max_M // PANEL), dtype=np.int64)

    def step(self, M, epoch):
        TM = M // PANEL
        C = tail_cols(M, tiles_n=self.tiles_n)
        self.panel_done[:, :TM] = 0
        for src in range(self.world):                       # producers: every rank scatters every tile
            for L in range(TM * self.tiles_n):
                m, n = remap_tile(L, TM, self.tiles_n, C)
                o, j = owner_of(m, self.world)
                self.tile_flags[o, src, j, n] = epoch
        for r in range(self.world):                         # owner reducers
            Pr = panels_owned(M, r, self.world)
            for u in range(Pr * self.tiles_n * QUARTERS):
                j, n, _q = unit_map(u, Pr, self.tiles_n, C)
                assert all(self.tile_flags[r, s, j, n] == epoch for s in range(self.world))
                m = j * self.world + r
                self.panel_done[r, m] += 1
                if self.panel_done[r, m] == self.tiles_n * QUARTERS:
                    self.panel_flag[:, m] = epoch


# ---------------------------------------------------------------------------------------- arithmetic
def make_weights(seed=0, K=K_FFN, N2_=N2, n1=N1):
    """Full weights, bf16, on the CPU: Wdown (n1, K) ~ N(0, 1/K), gamma (n1) ~ U(0.5, 1.5), Wqkv (N2_, n1) ~ N(0, 1/n1)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    Wd = (torch.randn(n1, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    gamma = (0.5 + torch.rand(n1, generator=g)).to(torch.bfloat16)
    Wq = (torch.randn(N2_, n1, generator=g) * n1 ** -0.5).to(torch.bfloat16)
    return Wd, gamma, Wq


def make_inputs(M, seed=1, K=K_FFN, n1=N1):
    """h (M, K) ~ N(0,1) and resid (M, n1) ~ N(0,1), bf16, CPU."""
    import torch
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(M, K, generator=g).to(torch.bfloat16)
    resid = torch.randn(M, n1, generator=g).to(torch.bfloat16)
    return h, resid


def shard_weights(Wdown, Wqkv, gamma, rank, world):
    """(Wdown column shard, Wqkv row shard, Wqkv row shard with gamma folded)   (ctapp/tp4.py:38-44)."""
    import torch
    Kr, N2r = Wdown.shape[1] // world, Wqkv.shape[0] // world
    Wd = Wdown[:, rank * Kr:(rank + 1) * Kr].contiguous()
    Wq = Wqkv[rank * N2r:(rank + 1) * N2r].contiguous()
    return Wd, Wq, fold_gamma(Wq, gamma)


def fold_gamma(Wq, gamma):
    """bf16( fp32(Wq) * fp32(gamma)[None, :] )   (ctapp/tp4.py:53-56)."""
    import torch
    return (Wq.float() * gamma.float()[None, :]).to(torch.bfloat16).contiguous()


def boundary_reference(h_full, Wdown_full, resid, gamma, Wqkv_full, eps=EPS):
    """fp32 chain -> (x_new fp32 (M, n1), out fp32 (M, N2))   (ctapp/tp4.py:650-656)."""
    import torch
    with torch.no_grad():
        x = h_full.float() @ Wdown_full.float().t()
        if resid is not None:
            x = x + resid.float()
        n = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()
        return x, n @ Wqkv_full.float().t()


def boundary_device_model(h_full, Wdown_full, resid, gamma, Wqkv_full, world, eps=EPS):
    """The rounding sequence of the device path, on the CPU: per-rank partial = bf16(fp32 GEMM); x = bf16(p0 + p1 +
    ... + resid) added left to right in fp32; rowss = sum of squares of the ROUNDED x; out_r = bf16((x @ Wf_r^T) *
    rsqrt(rowss / n1 + eps)).  Returns (x bf16, out bf16 with the rank shards concatenated)."""
    import torch
    with torch.no_grad():
        n1 = Wdown_full.shape[0]
        Kr = Wdown_full.shape[1] // world
        acc = None
        for r in range(world):
            p = (h_full[:, r * Kr:(r + 1) * Kr].float() @ Wdown_full[:, r * Kr:(r + 1) * Kr].float().t()).to(torch.bfloat16).float()
            acc = p if acc is None else acc + p
        if resid is not None:
            acc = acc + resid.float()
        x = acc.to(torch.bfloat16)
        rowss = x.float().pow(2).sum(-1, keepdim=True)
        scale = torch.rsqrt(rowss / n1 + eps)
        Wf = fold_gamma(Wqkv_full, gamma)
        out = ((x.float() @ Wf.float().t()) * scale).to(torch.bfloat16)
        return x, out


def silu_and_mul(g):
    """(M, 2 I) bf16 -> (M, I) bf16: silu(g[:, :I]) * g[:, I:], computed in fp32 on the bf16 inputs and rounded once: the
    activation between the gate/up and the down projection, which the reference leaves to the serving stack
    (vllm_plugin/ctapp_vllm/model.py:183, ``mlp.act_fn``) and names as a candidate for fusion into the GEMM epilogue
    (PLAN.md:597).  Restated from the published definition silu(x) = x / (1 + exp(-x))."""
    import torch
    I = g.shape[1] // 2
    a, b = g[:, :I].float(), g[:, I:].float()
    return (a / (1.0 + torch.exp(-a)) * b).to(torch.bfloat16)
