"""Llama-70B-architecture tensor-parallel prefill with both all-reduce boundaries of every layer CTA-pipelined.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node T --master-addr 127.0.0.1 --master-port P \
        cta-pipelining_b200/bench/llama_prefill.py [--layers 80] [--tokens 4096] [--batch 1] [--iters 5] [--check 2] \
        [--act kernel|fused|eager]

Architecture: hidden 8192, 64 query / 8 key-value heads of 128, FFN 28672 SwiGLU, RMSNorm eps 1e-5, rotary positions,
random-init bf16 weights (layer l from seed 1000 + l, fan-in scaled), seeded random token ids.  Standalone: attention is
torch SDPA, no serving engine.  Two paths over the same weights:
  stock      o_proj / down_proj with cuBLAS, NCCL all-reduce, one fused add+RMSNorm kernel, next projection with cuBLAS
  pipelined  boundary A (o_proj -> reduce + residual + RMSNorm -> gate_up) and boundary B (down_proj -> ... -> next layer's
             QKV) through ``ctapp.tp4.CtappBoundary``; layer 0's QKV and the last layer's down_proj stay stock
SwiGLU (``--act``): "kernel" = one silu-and-mul pass in both paths (``ctapp_silu_mul``, what a serving stack runs);
"fused" = the pipelined path applies it in boundary A's consumer epilogue (gate/up rows interleaved), the stock path keeps
the kernel; "eager" = torch ops in both paths.
The RMSNorm gammas are folded into the consuming weights (QKV, gate_up) for both paths, so the stock norm runs with a
weight of ones: both paths then compute the same function and can be compared layer by layer (``--check N`` layers).
Replaces the reference's vLLM-based drivers (bench/vllm_prefill.py, bench/vllm_ctapp_check.py) for boxes without the model
files or the serving engine.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
import torch.nn.functional as F  # noqa: E402

from ctapp import tp4  # noqa: E402

HIDDEN, HQ, HKV, HD, FFN, EPS = 8192, 64, 8, 128, 28672, 1e-5


class Layer:
    """One decoder layer's weight shards of rank ``r`` (gammas already folded into qkv and gate_up)."""

    def __init__(self, l, r, t, dev, fuse_act=False):
        g = torch.Generator(device=dev).manual_seed(1000 + l)     # same stream on every rank; each keeps its shard
        def w(rows, cols):
            return (torch.randn(rows, cols, generator=g, device=dev, dtype=torch.float32) * cols ** -0.5)
        g_in = 0.5 + torch.rand(HIDDEN, generator=g, device=dev)
        g_post = 0.5 + torch.rand(HIDDEN, generator=g, device=dev)
        hq, hkv = HQ // t, max(HKV // t, 1)
        # fused QKV rows of this rank: its query heads, its key heads, its value heads
        wq = w(HQ * HD, HIDDEN)[r * hq * HD:(r + 1) * hq * HD]
        kv_r = (r * HKV) // t
        wk = w(HKV * HD, HIDDEN)[kv_r * HD:(kv_r + hkv) * HD]
        wv = w(HKV * HD, HIDDEN)[kv_r * HD:(kv_r + hkv) * HD]
        self.qkv = (torch.cat([wq, wk, wv]) * g_in[None, :]).to(torch.bfloat16).contiguous()
        self.o = w(HIDDEN, HQ * HD)[:, r * hq * HD:(r + 1) * hq * HD].to(torch.bfloat16).contiguous()
        f = FFN // t
        gate = w(FFN, HIDDEN)[r * f:(r + 1) * f]
        up = w(FFN, HIDDEN)[r * f:(r + 1) * f]
        self.gate_up = (torch.cat([gate, up]) * g_post[None, :]).to(torch.bfloat16).contiguous()
        self.gate_up_i = tp4.interleave_gate_up(self.gate_up) if fuse_act else None     # for the activation epilogue
        self.down = w(HIDDEN, FFN)[:, r * f:(r + 1) * f].to(torch.bfloat16).contiguous()
        self.hq, self.hkv, self.f = hq, hkv, f


def rope_tables(S, dev):
    inv = 1.0 / (500000.0 ** (torch.arange(0, HD, 2, device=dev, dtype=torch.float32) / HD))
    ang = torch.arange(S, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cos(ang), torch.sin(ang)


def rope(x, cos, sin):          # x (B, H, S, D)
    x1, x2 = x[..., : HD // 2].float(), x[..., HD // 2:].float()
    c, s = cos[None, None], sin[None, None]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def attention(qkv, L, B, S, cos, sin):
    """qkv (B*S, (hq + 2 hkv) * 128) -> (B*S, hq * 128), causal, grouped-query."""
    q, k, v = qkv.split([L.hq * HD, L.hkv * HD, L.hkv * HD], dim=-1)
    q = q.view(B, S, L.hq, HD).transpose(1, 2)
    k = k.view(B, S, L.hkv, HD).transpose(1, 2)
    v = v.view(B, S, L.hkv, HD).transpose(1, 2)
    q, k = rope(q, cos, sin), rope(k, cos, sin)
    o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    return o.transpose(1, 2).reshape(B * S, L.hq * HD).contiguous()




class Model:
    def __init__(self, rank, t, dev, n_layers, max_M, fusion, act="kernel"):
        self.rank, self.t, self.dev, self.act = rank, t, dev, act
        self.layers = [Layer(l, rank, t, dev, act == "fused") for l in range(n_layers)]
        g = torch.Generator(device=dev).manual_seed(7)
        self.embed = (torch.randn(32000, HIDDEN, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        self.ones = torch.ones(HIDDEN, dtype=torch.bfloat16, device=dev)
        self.ext = tp4.load_tp4()
        L0 = self.layers[0]
        self.ba = tp4.CtappBoundary(max_M, L0.o.shape[1], L0.gate_up.shape[0], rank, t, None, dev, protocol="v5", max_M=max_M, fusion=fusion, qkv_raster=3, qkv_swizzle=4,
                                    down_tail=HIDDEN // 256, act=act == "fused")     # short producer (K = 8192 / t): panel-major, so panels complete one by one
        self.bb = tp4.CtappBoundary(max_M, L0.down.shape[1], L0.qkv.shape[0], rank, t, None, dev, protocol="v5", max_M=max_M, fusion=fusion)
        self.y = torch.empty(max_M, HIDDEN, dtype=torch.bfloat16, device=dev)
        self.xn = torch.empty(max_M, HIDDEN, dtype=torch.bfloat16, device=dev)
        self.xo = [torch.empty(max_M, HIDDEN, dtype=torch.bfloat16, device=dev) for _ in range(2)]

    def swiglu(self, g, f):
        if self.act == "eager":
            return (F.silu(g[:, :f].float()) * g[:, f:].float()).to(g.dtype)
        return self.ext.silu_mul(g)

    def stock_boundary(self, a, resid, Wd, Wq, k):
        """cuBLAS GEMM + NCCL all-reduce + fused add-RMSNorm (ones weight: gamma lives in Wq) + cuBLAS GEMM -> (out, x)."""
        M = a.shape[0]
        torch.mm(a, Wd.t(), out=self.y[:M])
        if self.t > 1:
            dist.all_reduce(self.y[:M])
        self.ext.add_rmsnorm(self.y[:M], resid, self.ones, self.xo[k][:M], self.xn[:M], eps=EPS)
        return torch.mm(self.xn[:M], Wq.t()), self.xo[k][:M]

    def forward(self, ids, B, S, pipelined, check=0, log=None):
        cos, sin = rope_tables(S, self.dev)
        x = self.embed[ids]                                   # residual stream (B*S, 8192)
        h = tp4.rmsnorm_gamma(x, self.ones, EPS)
        qkv = torch.mm(h, self.layers[0].qkv.t())
        n = len(self.layers)
        for i, L in enumerate(self.layers):
            a = attention(qkv, L, B, S, cos, sin)
            if pipelined:
                if i < check:
                    g_ref, x_ref = self.stock_boundary(a, x, L.o, L.gate_up, 0)
                    g_ref, x_ref = g_ref.clone(), x_ref.clone()
                fused = self.act == "fused"
                g = self.ba.forward(a, x, L.o, L.gate_up_i if fused else L.gate_up)      # fused: already silu(gate) * up
                x = self.ba.x()
                if i < check and log is not None:
                    log.append((i, "A", rel(g, self.swiglu(g_ref, L.f) if fused else g_ref), rel(x, x_ref)))
                h_r = g if fused else self.swiglu(g, L.f)
            else:
                g, x = self.stock_boundary(a, x, L.o, L.gate_up, 0)
                h_r = self.swiglu(g, L.f)
            if i + 1 < n:
                nxt = self.layers[i + 1]
                if pipelined:
                    if i < check:
                        q_ref, x_ref = self.stock_boundary(h_r, x, L.down, nxt.qkv, 1)
                        q_ref, x_ref = q_ref.clone(), x_ref.clone()
                    qkv = self.bb.forward(h_r, x, L.down, nxt.qkv)
                    x = self.bb.x()
                    if i < check and log is not None:
                        log.append((i, "B", rel(qkv, q_ref), rel(x, x_ref)))
                else:
                    qkv, x = self.stock_boundary(h_r, x, L.down, nxt.qkv, 1)
            else:                                             # last layer: stock down_proj + all-reduce + final norm
                y = torch.mm(h_r, L.down.t())
                if self.t > 1:
                    dist.all_reduce(y)
                x = y + x
        return tp4.rmsnorm_gamma(x, self.ones, EPS)


def rel(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=80)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--check", type=int, default=2, help="compare the first N layers' boundaries with the stock path")
    ap.add_argument("--fusion", default="pdl")
    ap.add_argument("--act", default="kernel", choices=["kernel", "fused", "eager"])
    a = ap.parse_args()
    rank, t = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if t > 1:
        dist.init_process_group("nccl", device_id=dev)
    else:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29578")
        dist.init_process_group("gloo", rank=0, world_size=1)
    tp4.GLOO = dist.new_group(backend="gloo")
    B, S = a.batch, a.tokens
    M = B * S
    assert M % 128 == 0 and HQ % t == 0 and FFN % t == 0
    model = Model(rank, t, dev, a.layers, M, a.fusion, a.act)
    ids = torch.tensor([random.Random(0).randint(1000, 31999) for _ in range(M)], device=dev)
    with torch.no_grad():
        log = []
        out_p = model.forward(ids, B, S, True, a.check, log).clone()
        model.ba.check(); model.bb.check()
        out_s = model.forward(ids, B, S, False).clone()
        torch.cuda.synchronize(dev)
        final_rel = rel(out_p, out_s)

        def timed(pipelined):
            ts = []
            for _ in range(a.iters):
                tp4.barrier(); torch.cuda.synchronize(dev)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); model.forward(ids, B, S, pipelined); e1.record()
                torch.cuda.synchronize(dev)
                ts.append(e0.elapsed_time(e1))
            v = torch.tensor([statistics.median(ts)], dtype=torch.float64)
            dist.all_reduce(v, op=dist.ReduceOp.MAX, group=tp4.GLOO)
            return float(v.item())
        model.forward(ids, B, S, True); model.forward(ids, B, S, False)
        ms_s, ms_p = timed(False), timed(True)
        model.ba.check(); model.bb.check()
    if rank == 0:
        print(json.dumps({"workload": f"Llama-70B-shape prefill, {a.layers} layers, TP{t}, batch {B} x {S} tokens", "act": a.act, "stock_ms": round(ms_s, 3),
                          "pipelined_ms": round(ms_p, 3), "speedup": round(ms_s / ms_p, 4), "final_hidden_rel_vs_stock": final_rel,
                          "per_layer_check": [dict(layer=i, boundary=b, out_rel=round(o, 5), x_rel=round(x, 5)) for i, b, o, x in log]}), flush=True)
    tp4.barrier()


if __name__ == "__main__":
    main()
