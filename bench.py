#!/usr/bin/env python
"""Benchmark of the CTA-pipelined layer-per-GPU GEMM chain.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens M]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload: an N-stage chain of bf16 linear layers, one stage per GPU, M = 8192 tokens, N = K = 8192, no activation,
X ~ N(0,1), W_l ~ N(0, 1/K), seeded, fp32 accumulation, bf16 between stages.  Stage g's output tiles are stored straight
into GPU g+1's memory by the GEMM epilogue and announced in that GPU's work queue; nothing else moves data.  At N = 1 the
chain is one stage: one 8192^3 GEMM through the same work-queue protocol.  A step is one run of the whole chain.

Prints ONE JSON line (rank 0): metric = chain TFLOP/s = N * 2*M*N*K / step time, whole job.  ``value`` is measured with the
inputs resident in HBM; ``e2e`` is the same through the public API with X in pinned host memory (copied in every step) and
the last stage's output copied back every step.  ``roofline`` is for the GEMM kernel (tensor-core bound), timed by CUDA
events around each launch.  ``cpu_baseline`` / ``--impl reference`` time the reference's torch CPU path (fp32 ``F.linear``
chain) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "cta-pipelining_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

NK = 8192
GEMM_CFG = 10        # CTA-pair tcgen05 kernel, 256 x 256 x 64 tiles (two TMEM accumulators)
GEMM_CFG_WIDE = 11   # the same kernel on 256 x 512 x 64 tiles (one TMEM accumulator, a quarter less operand traffic)
CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
               "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
# measured DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum of one launch under ncu) per configuration id, captured on
# an M = 2048 launch of the same kernel: {"<cfg>": {"M": 2048, "bytes": ...}}; traffic grows in proportion to M
TRAFFIC_FILE = os.path.join(ROOT, "cta-pipelining_b200", "bench", "ncu_traffic.json")


def dram_traffic(cfg, M):
    try:
        rec = json.load(open(TRAFFIC_FILE)).get(str(cfg))
        return int(rec["bytes"] * M / rec["M"]) if rec else None
    except (OSError, ValueError, KeyError):
        return None


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("bf16_tflops"), d.get("bf16_tflops_sustained"), "measured"
    return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx = float(r[2])
                for name, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        busy = [c for c in sm if mx and c > 0.3 * mx] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def cpu_chain_reference(M, n_stages, reps, threads=None):
    """The reference's CPU path for this workload: fp32 F.linear per stage, bf16 between stages.  Returns (best s, TFLOP/s)."""
    from oracle import chain as oc
    if threads:
        torch.set_num_threads(threads)
    X, Ws = oc.make_chain_inputs(M, NK, [NK] * n_stages, seed=0)
    best = float("inf")
    for _ in range(reps):
        t = time.perf_counter()
        oc.chain_reference(X, Ws)
        best = min(best, time.perf_counter() - t)
    return best, n_stages * 2 * M * NK * NK / best / 1e12


def run_reference(args, rank):
    """--impl reference: the reference's own CPU implementation of the path, on all host cores."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    M_s = args.m                                # the whole workload: every token row through every stage, every step
    n = max(args.gpus, 1)
    ts = []
    from oracle import chain as oc
    torch.set_num_threads(cores)
    X, Ws = oc.make_chain_inputs(M_s, NK, [NK] * n, seed=0)
    for i in range(args.warmup + args.steps):
        t = time.perf_counter()
        oc.chain_reference(X, Ws)
        dt = time.perf_counter() - t
        if i >= args.warmup:
            ts.append(dt)
    ms = statistics.mean(ts) * 1e3
    val = n * 2 * M_s * NK * NK / (ms * 1e-3) / 1e12
    line = {"impl": "reference", "metric": "chain_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(args, n),
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": f"all {M_s} token rows, all {n} stages, torch CPU fp32 F.linear chain, {args.steps} steps"},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(args, n):
    if args.scoreboard == "auto":
        args.scoreboard = "kchunk"
    if args.cfg == "auto":
        args.cfg = GEMM_CFG_WIDE
    args.cfg = int(args.cfg)
    return {"workload": f"{n}-stage layer-per-GPU bf16 linear chain, M={args.m} tokens, N=K={NK}, no activation, one stage per GPU"
                        + (" (N=1: one GEMM through the work-queue protocol)" if n == 1 else ""),
            "M": args.m, "N": NK, "K": NK, "stages": n, "tile": {10: "256x256x64 per CTA pair (cta_group::2)", 11: "256x512x64 per CTA pair (cta_group::2, one TMEM accumulator)",
                                                                       3: "128x256x64 per CTA"}[args.cfg], "parallelism": f"pp{n}",
            "l2": "inputs larger than L2 (X, W, Y are 3 x 128 MiB per stage)",
            "dependencies": "none (one stage)" if n == 1 else ("row-panel scoreboard + work queue" if args.scoreboard == "rowpanel" else "k-chunk value flags"),
            "steps_overlap": "none (one GEMM per step)" if n == 1 else
            "consecutive steps stream through the stages like batches through a layer pipeline: every link (buffer, queue, "
            "ready flag) is doubled, so a stage starts step e+1 while its successor still consumes step e; at most two steps "
            "in flight per link; ms_per_step is the K steps' total time / K, fill included"}


def _init_groups(world, dev, port):
    """NCCL default group + gloo side group for the stand-alone workloads (idempotent)."""
    import torch.distributed as dist
    from ctapp import tp4
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if not dist.is_initialized():
        if world > 1:
            dist.init_process_group("nccl", device_id=dev)
        else:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", str(port))
            dist.init_process_group("gloo", rank=0, world_size=1)
    if tp4.GLOO is None:
        tp4.GLOO = dist.new_group(backend="gloo")


def boundary_record(args, rank, world, dev, M=None, with_eager=True):
    """TP layer boundary at TP = world: down-proj partial GEMM (K = 28672 / t, N = 8192, M tokens) -> cross-rank sum + bf16
    residual + RMSNorm (eps 1e-5) -> QKV GEMM (K = 8192, N = 10240 / t).  Times the CTA-pipelined boundary, its two-GEMM floor,
    and the stock boundary (cuBLAS GEMM + NCCL all-reduce + one fused add+RMSNorm kernel + cuBLAS GEMM); back-to-back mean and
    per-step median, max over ranks.  Process groups must be up.  Returns the record (rank 0) or None."""
    import torch.distributed as dist
    from ctapp import tp4
    M = M or args.m
    t = world
    Kr, N2r = (tp4.K_FFN // t, tp4.N2 // t) if args.shape == "B" else (8192 // t, 57344 // t)
    if args.shard_as:      # the per-rank shapes of a wider tensor-parallel group on this many GPUs (a TP8 rank's GEMMs with a TP4 exchange)
        Kr, N2r = tp4.K_FFN // args.shard_as, tp4.N2 // args.shard_as
    kfull = Kr * t
    akw = {} if args.shape == "B" else dict(qkv_raster=3, qkv_swizzle=4, down_tail=tp4.N1 // 256)
    g = torch.Generator().manual_seed(0)
    # per-rank shards drawn directly (the full 28672-wide weights never exist in one place; parity is covered by the tests)
    Wd_r = (torch.randn(tp4.N1, Kr, generator=g) * kfull ** -0.5).to(torch.bfloat16).to(dev)
    gamma = (0.5 + torch.rand(tp4.N1, generator=g)).to(torch.bfloat16).to(dev)
    Wq_r = (torch.randn(N2r, tp4.N1, generator=g) * tp4.N1 ** -0.5).to(torch.bfloat16).to(dev)
    Wqf_r = tp4.fold_gamma(Wq_r, gamma)
    h_r = torch.randn(M, Kr, generator=g).to(torch.bfloat16).to(dev)
    resid = torch.randn(M, tp4.N1, generator=g).to(torch.bfloat16).to(dev)
    iters, warm = max(args.steps, 10), max(args.warmup, 3)
    res = {}
    steal = args.steal == 1
    bd = tp4.CtappBoundary(M, Kr, N2r, rank, t, None, dev, protocol=args.protocol if t > 1 else "v5", max_M=M, fusion=args.fusion,
                           R=None if args.R < 0 else args.R, steal=steal, red_blocks=args.red_blocks if args.red_blocks >= 0 else None,
                           red_threads=args.red_threads, cta_pair={1: "wide", 0: "narrow"}.get(args.down_wide, True), **akw)
    bd.set_weights(Wd_r, Wqf_r)
    res["ctapp"] = tp4.time_step(lambda: bd.forward(h_r, resid), dev, iters, warm)
    bd.check()
    fl = tp4.CtappBoundary(M, Kr, N2r, rank, t, None, dev, protocol=False, max_M=M, R=bd.R, red_blocks=1, cta_pair={1: "wide", 0: "narrow"}.get(args.down_wide, True), **akw)
    res["two_gemm_floor"] = tp4.time_step(lambda: fl.forward(h_r, None, Wd_r, Wqf_r), dev, iters, warm)
    st = tp4.NcclFusedNormBoundary(M, rank, t, None, dev, Wd_r, Wq_r, gamma)
    res["cublas_nccl_fusednorm"] = tp4.time_step(lambda: st.forward(h_r, resid), dev, iters, warm)
    if with_eager:
        st2 = tp4.NcclBoundary(M, rank, t, None, dev, Wd_r, Wq_r, gamma)
        res["cublas_nccl_eagernorm"] = tp4.time_step(lambda: st2.forward(h_r, resid), dev, iters, warm)
    unavailable = {}
    if args.baselines == "strong" and t > 1:
        for name, cls in (("cublas_multimem_ar_eagernorm", tp4.MultimemBoundary), ("asynctp_matmul_reduce_scatter", tp4.AsyncTpBoundary)):
            try:
                bs = cls(M, rank, t, None, dev, Wd_r, Wq_r, gamma)
                res[name] = tp4.time_step(lambda: bs.forward(h_r, resid), dev, iters, warm)
            except Exception as e:  # noqa: BLE001  (a baseline that this torch build cannot run is reported, not fatal)
                unavailable[name] = repr(e)[:200]
            ok_all = torch.tensor([0 if name in unavailable else 1])
            dist.all_reduce(ok_all, op=dist.ReduceOp.MIN, group=tp4.GLOO)
            if not int(ok_all.item()):
                res.pop(name, None)
                unavailable.setdefault(name, "failed on another rank")
    # agreement of the two paths on this rank's output shard (bf16 tolerance; different rounding points)
    o1 = bd.forward(h_r, resid).float(); o2 = st.forward(h_r, resid).float()
    torch.cuda.synchronize(dev)
    rel = float((o1 - o2).abs().max() / o2.abs().max())
    tp4.barrier()
    if rank != 0:
        return None
    flops = 2 * M * Kr * tp4.N1 + 2 * M * tp4.N1 * N2r
    burst, sustained, kind = peaks()
    b2b = res["ctapp"][1]
    return {"workload": f"TP{t} layer boundary {args.shape}, M={M}, producer K={Kr} N=8192 -> reduce + residual + RMSNorm -> consumer N={N2r}",
            "n_gpus": t, "fusion": args.fusion, "steal": steal, "R": bd.R, "red_blocks": bd.red_blocks, "red_threads": bd.red_threads, "producer_tile": "256x512" if bd.down_pair(M) == 2 else "256x256", "push": ("nvls multimem + in-switch reduction" if bd.ldreduce else "nvls multimem") if bd.nvls else "unicast",
            "ms_median_b2b": {k: [round(v[0], 4), round(v[1], 4)] for k, v in res.items()},
            "speedup_vs_cublas_nccl_fusednorm_b2b": res["cublas_nccl_fusednorm"][1] / b2b,
            "over_two_gemm_floor_b2b": b2b / res["two_gemm_floor"][1],
            "tflops_per_gpu_b2b": flops / (b2b * 1e-3) / 1e12, "frac_of_burst_peak": flops / (b2b * 1e-3) / 1e12 / burst,
            "out_rel_vs_stock": rel, "iters": iters, "unavailable": unavailable}


def run_boundary(args, rank, world, local_rank):
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    _init_groups(world, dev, 29577)
    rec = boundary_record(args, rank, world, dev)
    if rank == 0:
        print(json.dumps(rec), flush=True)


def latency_record(M_list, cfg, reps=10):
    """Gated single-run latency of the two-stage chain on GPUs 0 and 1, driven from this one process (the other ranks idle at a
    barrier): the north-star figure, chain time over the ideal = one library GEMM's time (both layers on one GPU / 2), beside
    micro-batched library GEMMs with peer copies.  Mirrors reference bench/fig5.py:29-93 for the M given."""
    from ctapp import methods as mt
    from ctapp.timing import measure
    g = torch.Generator().manual_seed(0)
    W1 = (torch.randn(NK, NK, generator=g) / NK ** 0.5).to(torch.bfloat16)
    W2 = (torch.randn(NK, NK, generator=g) / NK ** 0.5).to(torch.bfloat16)
    W1a, W2a, W2b = W1.to(mt.dev(0)), W2.to(mt.dev(0)), W2.to(mt.dev(1))
    rows = []
    for M in M_list:
        X = torch.randn(M, NK, generator=g).to(torch.bfloat16).to(mt.dev(0))
        r = {"M": M}
        r["ideal_us"] = measure(mt.OneGpuCublas(M, X, W1a, W2a), reps, devs=(0,))[0] / 2
        r["ours_one_gpu_half_us"] = measure(mt.OneGpuTma(M, X, W1a, W2a, cfg), reps, devs=(0,))[0] / 2
        best = None
        for chunk in (512, 1024):
            t = measure(mt.MicroBatchCublas(M, X, W1a, W2b, chunk), reps)[0]
            best = (t, chunk) if best is None or t < best[0] else best
        r["microbatch_cublas_us"], r["microbatch_chunk"] = best
        # the reference's row-panel scoreboard at its best group size, and k-chunk dependencies with the consumer on the
        # 256 x 512 tile (one acquiring poll per 3.1 us of tensor work; on the 256 x 256 tile the polls starve the loader)
        for name, kw in (("rowpanel_g2", dict(group_rows=2)), ("kchunk_wide_consumer_g4", dict(group_rows=4, scoreboard="kchunk", cfg_c=GEMM_CFG_WIDE)),
                         ("kchunk_wide_consumer_g3", dict(group_rows=3, scoreboard="kchunk", cfg_c=GEMM_CFG_WIDE))):
            c = mt.Ctapp(M, X, W1a, W2b, cfg, kw.get("cfg_c", cfg), kw["group_rows"], scoreboard=kw.get("scoreboard", "rowpanel"))
            r[f"chain_{name}_us"] = measure(c, reps)[0]
            c.pl.check()
            del c
        r["chain_us"] = min(v for k, v in r.items() if k.startswith("chain_"))
        r["over_ideal"] = r["chain_us"] / r["ideal_us"]
        r["vs_microbatch"] = r["microbatch_cublas_us"] / r["chain_us"]
        rows.append({k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()})
        del X
        torch.cuda.empty_cache()
    return rows


def run_reducer(args, rank, world, local_rank):
    """The owner reducer alone (every tile flag already raised): reads the t inbox slices + the residual of this rank's M/t
    rows, writes x to every rank, publishes row sums and panel flags.  Bytes per rank with S = (M/t) * n1 * 2: HBM reads
    (t + 1) * S, HBM writes t * S (its own copy + what the peers push), NVLink egress (t - 1) * S.  One JSON line on rank 0."""
    import torch.distributed as dist
    from ctapp import tp4
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    _init_groups(world, dev, 29579)
    M, t = args.m, world
    out = {}
    rv = {}
    resid = torch.randn(M, tp4.N1, device=dev).to(torch.bfloat16)
    for R in ([args.R] if args.R > 0 else [4, 8, 16, 32]):
        bd = tp4.CtappBoundary(M, 256, 256, rank, t, None, dev, protocol=args.protocol if t > 1 else "v5", max_M=M, R=R, **rv)
        bd.inbox.normal_()
        ext = bd.ext
        times = []
        for it in range(max(args.warmup, 3) + max(args.steps, 10)):
            bd.epoch += 1
            ext.tp4_step(bd.epoch_dev, bd.rowss_local, bd.panel_done, M, bd.role_ctr)
            bd.tile_flags.fill_(bd.epoch)                      # every producer tile "has arrived"
            torch.cuda.synchronize(dev); tp4.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); bd.launch_reducer(M, resid, bd.epoch & 1); b.record()
            torch.cuda.synchronize(dev); tp4.barrier()
            if it >= max(args.warmup, 3):
                times.append(a.elapsed_time(b))
        bd.check()
        assert bool((bd.panel_flag[:M // 128].cpu() == bd.epoch).all())
        v = torch.tensor([statistics.median(times)], dtype=torch.float64)
        dist.all_reduce(v, op=dist.ReduceOp.MAX, group=tp4.GLOO)
        out[R] = float(v.item())
        del bd
    if rank == 0:
        S = (M // t) * tp4.N1 * 2
        peak_hbm = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("hbm_gbs", 6650.0) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 6650.0
        rows = {}
        for R, ms in out.items():
            hbm = ((t + 1) * S + t * S) / (ms * 1e-3) / 1e9
            link = (t - 1) * S / (ms * 1e-3) / 1e9
            rows[R] = {"ms": round(ms, 4), "hbm_GBs": round(hbm, 1), "hbm_frac_of_measured_peak": round(hbm / peak_hbm, 4),
                       "nvlink_egress_GBs": round(link, 1), "nvlink_frac_of_770": round(link / 770.0, 4)}
        print(json.dumps({"workload": f"owner reducer alone, TP{t}, M={M}, n1=8192, push={'nvls' if args.protocol == 'v3' and t > 1 else 'unicast'}",
                          "bytes_per_rank": {"hbm_read": (t + 1) * S, "hbm_write": t * S, "nvlink_egress": (t - 1) * S}, "by_R": rows}), flush=True)
    tp4.barrier()


def run_stages(args, rank, world, local_rank):
    """Stage breakdown of the boundary (what reference bench/v5_stages.py:40-277 reports): the producer GEMM storing locally
    (mode 0) and scattering to the owners with flags (mode 7), the owner reducer alone, the consumer GEMM plain (mode 0) and
    waiting per panel on flags that are already up (mode 5), and the whole boundary; back-to-back mean ms, max over ranks.  The
    scatter's NVLink egress is (t - 1) / t of the producer's output."""
    import torch.distributed as dist
    from ctapp import tp4
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    _init_groups(world, dev, 29580)
    M, t = args.m, world
    Kr, N2r = (tp4.K_FFN // t, tp4.N2 // t) if args.shape == "B" else (8192 // t, 57344 // t)
    akw = {} if args.shape == "B" else dict(qkv_raster=3, qkv_swizzle=4, down_tail=tp4.N1 // 256)
    g = torch.Generator().manual_seed(0)
    Wd = (torch.randn(tp4.N1, Kr, generator=g) * (Kr * t) ** -0.5).to(torch.bfloat16).to(dev)
    Wq = (torch.randn(N2r, tp4.N1, generator=g) * tp4.N1 ** -0.5).to(torch.bfloat16).to(dev)
    h = torch.randn(M, Kr, generator=g).to(torch.bfloat16).to(dev)
    resid = torch.randn(M, tp4.N1, generator=g).to(torch.bfloat16).to(dev)
    bd = tp4.CtappBoundary(M, Kr, N2r, rank, t, None, dev, protocol=args.protocol if t > 1 else "v5", max_M=M, fusion=args.fusion, R=None if args.R < 0 else args.R, **akw)
    ext, iters = bd.ext, max(args.steps, 10)
    y0 = torch.empty(M, tp4.N1, dtype=torch.bfloat16, device=dev)

    def b2b(fn, prep=None):
        for _ in range(3):
            if prep:
                prep()
            fn()
        torch.cuda.synchronize(dev); tp4.barrier()
        ts = []
        for _ in range(iters):          # each call bracketed: stages that wait for peers must start together
            if prep:
                prep()
            torch.cuda.synchronize(dev); tp4.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize(dev)
            ts.append(a.elapsed_time(b))
        v = torch.tensor([statistics.median(ts)], dtype=torch.float64)
        dist.all_reduce(v, op=dist.ReduceOp.MAX, group=tp4.GLOO)
        return float(v.item())

    def step():
        bd.epoch += 1
        ext.tp4_step(bd.epoch_dev, bd.rowss_local, bd.panel_done, M, bd.role_ctr)

    res = {}
    res["producer_mode0_local"] = b2b(lambda: ext.tp4_down(h, Wd, y0, 1, 1, 0, rank, t, 0, sms=bd.sms, tail_cols=bd.tail_cols(M), cta_pair=bd.cta_pair))
    res["producer_mode7_scatter"] = b2b(lambda: bd.launch_producer(h, Wd, M), step)
    res["reducer_alone"] = b2b(lambda: bd.launch_reducer(M, resid, bd.epoch & 1))            # flags of the last scatter are still up
    res["consumer_mode0"] = b2b(lambda: ext.tp4_qkv(bd.xbufs[bd.epoch & 1][:M], Wq, bd._out_full[:M], bd.qkv_raster, bd.qkv_swizzle, 0, 0, sms=bd.qkv_sms,
                                                   tile=bd.qkv_tile, cta_pair=bd.cta_pair))
    res["consumer_mode5_flags_up"] = b2b(lambda: bd.launch_consumer(Wq, M, bd.epoch & 1))
    res["boundary"] = b2b(lambda: bd.forward(h, resid, Wd, Wq))
    bd.check()
    if rank == 0:
        out_bytes = M * tp4.N1 * 2
        egress = (t - 1) / t * out_bytes
        extra = max(res["producer_mode7_scatter"] - res["producer_mode0_local"], 1e-9)
        print(json.dumps({"workload": f"TP{t} boundary {args.shape} stage breakdown, M={M}, R={bd.R}, push={'nvls' if bd.nvls else 'unicast'}",
                          "ms": {k: round(v, 4) for k, v in res.items()},
                          "scatter": {"nvlink_egress_bytes": int(egress), "egress_GBs_over_kernel": round(egress / (res["producer_mode7_scatter"] * 1e-3) / 1e9, 1),
                                      "penalty_vs_local_store": round(res["producer_mode7_scatter"] / res["producer_mode0_local"], 4),
                                      "extra_ms": round(extra, 4)}}), flush=True)
    tp4.barrier()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cfg", default="auto", choices=["auto", "3", "10", "11"],
                    help="chain: GEMM configuration id (10 = CTA pair on 256x256x64 tiles, 11 = CTA pair on 256x512x64, 3 = one CTA on "
                    "128x256x64; auto = 11: it measured 5.5 %% faster on one GPU, 2-6 %% on two and 3 %% in the one-second loop on four)")
    ap.add_argument("--tokens", dest="m", type=int, default=None, help="M, the number of token rows (default 8192 for the chain, 4096 for the boundary)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="chain", choices=["chain", "boundary", "reducer", "stages"],
                    help="chain (default, the headline line) | boundary: TP layer boundary vs cuBLAS + NCCL all-reduce + fused norm")
    ap.add_argument("--scoreboard", default="auto", choices=["auto", "rowpanel", "kchunk"],
                    help="chain at N >= 2: how a stage learns that its input has arrived: the reference's row-panel scoreboard and work queue, or "
                    "k-chunk value flags (a tile's main loop streams behind the stage before it; auto: the fill a link adds is shorter, 20 steps "
                    "measured 0.755 against 0.763 ms per step on 2 GPUs and 0.789 against 0.807 on 4, the one-second loop the same)")
    ap.add_argument("--group-rows", default="auto", help="chain: tile rows the first stage walks together: an integer, 'ramp' (small groups first "
                    "and last, large in the middle), 'head' (groups of 2, 4, then 8 tile rows: the next stage starts after one wave) or 'auto' (8: 'head' "
                    "measured 0.7-0.9 %% slower on 2 GPUs and 0.2-1 %% slower on 4)")
    ap.add_argument("--fusion", default="pdl", choices=["none", "pdl", "pdl1", "role"])
    ap.add_argument("--steal", type=int, default=-1, help="boundary: 1 = the consumer's CTAs help the owner reducer (mode 8), 0 = off, -1 = off (the library's default): it measured neutral to slightly slower at TP2 and TP4")
    ap.add_argument("--shard-as", type=int, default=0, help="boundary: use the per-rank GEMM shapes of this tensor-parallel degree (0 = the launch's own)")
    ap.add_argument("--down-wide", type=int, default=-1, help="boundary: 1 = the producer GEMM works on 256 x 512 tiles, 0 = on 256 x 256, -1 = the library's choice")
    ap.add_argument("--red-blocks", type=int, default=-1, help="boundary: reducer CTAs (-1 = R; with --R 0 they share SMs with the GEMMs' CTAs)")
    ap.add_argument("--red-threads", type=int, default=1024, help="boundary: threads per reducer CTA (<= 512 to share an SM with a GEMM CTA)")
    ap.add_argument("--no-sustained", action="store_true", help="chain: keep the one-second sustained loop as short as the timed region (profiler captures)")
    ap.add_argument("--no-extras", action="store_true", help="chain: skip the gated-latency, boundary and oracle records that follow the timed regions")
    ap.add_argument("--protocol", default="v5", choices=["v5", "v3", "v3r"],
                    help="boundary: v5 = unicast pushes, v3 = NVLS multimem pushes, v3r = v3 + the cross-rank sum by multimem.ld_reduce inside the NVSwitch")
    ap.add_argument("--baselines", default="stock", choices=["stock", "strong"],
                    help="boundary: strong = also torch's multimem all-reduce and async-TP (fused matmul + reduce-scatter) boundaries")
    ap.add_argument("--shape", default="B", choices=["A", "B"], help="boundary: B = down-proj -> QKV (headline), A = o_proj -> gate_up")
    ap.add_argument("--R", type=int, default=-1, help="boundary: SMs reserved for the owner reducer (-1 = library default: 4 up to TP2, 8 at TP4, 12 at TP8; 0 with "
                    "--steal 1 = none, the consumer's CTAs do the reduction)")
    args = ap.parse_args()
    if args.m is None:
        args.m = 4096 if args.workload == "boundary" and args.impl == "ours" else 8192
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "boundary":
        run_boundary(args, rank, world, local_rank)
        return
    if args.workload == "reducer":
        run_reducer(args, rank, world, local_rank)
        return
    if args.workload == "stages":
        run_stages(args, rank, world, local_rank)
        return
    assert world == max(args.gpus, 1), f"--gpus {args.gpus} needs {args.gpus} ranks (torch.distributed.run), got WORLD_SIZE={world}"
    import torch.distributed as dist
    from ctapp.pipeline import Chain, ChainStage

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        gloo = dist.new_group(backend="gloo")
    M, n = args.m, world
    W_steps, K_steps = max(args.warmup, 3), args.steps
    flops_step = n * 2 * M * NK * NK

    def barrier():
        if world > 1:
            dist.barrier(group=gloo)

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=gloo)
        return float(t.item())

    # ---- inputs (seeded on the CPU; every rank draws the same stream and keeps its stage's weight)
    g = torch.Generator().manual_seed(0)
    X_host = torch.randn(M, NK, generator=g).to(torch.bfloat16).pin_memory() if rank == 0 else None
    if rank != 0:
        torch.randn(M, NK, generator=g)
    Wmine = None
    for s in range(n):
        w = torch.randn(NK, NK, generator=g)
        if s == rank:
            Wmine = (w / NK ** 0.5).to(torch.bfloat16).to(dev)
        del w
    X_dev = X_host.to(dev) if rank == 0 else None
    Y_host = torch.empty(M, NK, dtype=torch.bfloat16).pin_memory() if rank == n - 1 else None

    # measured at N = 4 (20-step / one-second figures, ms per step): 256x512 tiles in groups of 8: 0.811 / 0.880; 256x256 in groups
    # of 8: 0.810 / 0.906; 256x512 head-ramped: 0.813 / 0.891; 256x256 head-ramped: 0.829 / 0.927
    args.cfg = GEMM_CFG_WIDE if args.cfg == "auto" else int(args.cfg)
    if args.scoreboard == "auto":
        args.scoreboard = "kchunk"
    gr = args.group_rows
    gr = 8 if gr == "auto" else (gr if gr in ("ramp", "head") else int(gr))
    args.group_rows = gr
    if world == 1:
        chain = Chain(M, NK, [NK], [local_rank], cfg=args.cfg, group_rows=args.group_rows)
        step = lambda: chain.run(X_dev, [Wmine])  # noqa: E731
        checker = chain.check
        launches_per_step = 2   # reset kernel + GEMM kernel
    else:
        stage = ChainStage(M, NK, [NK] * n, rank, world, dev, group=None, cfg=args.cfg, group_rows=args.group_rows, scoreboard=args.scoreboard)
        step = lambda: stage.step(Wmine, X_dev)  # noqa: E731
        checker = stage.check
        launches_per_step = 2 * n

    # ---- device-resident timing: W warm-up steps, then exactly K steps between barriers
    for _ in range(W_steps):
        step()
    checker()
    barrier()
    torch.cuda.synchronize(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clk:
        barrier()
        torch.cuda.synchronize(dev)
        a.record()
        for _ in range(K_steps):
            step()
        b.record()
        torch.cuda.synchronize(dev)
        barrier()
        ms_total = max_over_ranks(a.elapsed_time(b))
        # the same steps for about a second more (same count on every rank): what the 100 ms clock sampler can see, and the
        # sustained figure at the power cap that goes with those clocks
        n_tail = K_steps if args.no_sustained else int(min(4000, 1000.0 / max(ms_total / K_steps, 0.05)))
        barrier()
        a_t, b_t = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a_t.record()
        for _ in range(n_tail):
            step()
        b_t.record()
        torch.cuda.synchronize(dev)
        barrier()
        sustained_ms = max_over_ranks(a_t.elapsed_time(b_t)) / n_tail
    checker()
    ms_step = ms_total / K_steps
    value = flops_step / (ms_step * 1e-3) / 1e12

    # ---- the GEMM kernel alone: CUDA events around each launch on the launching stream
    # (with more than one stage a stage's kernel spans the whole pipelined run, so its duration is the step's)
    kernel_ms = ms_step
    if world == 1:
        kt = []
        for _ in range(K_steps):
            chain.reset()
            a2, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a2.record(); chain.enqueue(X_dev, [Wmine]); b2.record()
            torch.cuda.synchronize(dev)
            kt.append(a2.elapsed_time(b2))
        checker()
        kernel_ms = statistics.mean(kt)

    # ---- end to end through the public API: every step copies X in from pinned host memory and the last stage's Y back out.
    # The copies of neighbouring steps overlap the compute (two device buffers each way, a copy-in and a copy-out stream), as
    # a caller that streams batches through the chain would arrange it; every byte still crosses the bus every step.
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    first_rank, last_rank = rank == 0, rank == n - 1
    xbufs = [X_dev, torch.empty_like(X_dev)] if first_rank else [None, None]
    ybufs = [torch.empty(M, NK, dtype=torch.bfloat16, device=dev) for _ in range(2)] if last_rank else None
    yhost = [Y_host, torch.empty(M, NK, dtype=torch.bfloat16).pin_memory()] if last_rank else None
    ev = {k: [torch.cuda.Event(), torch.cuda.Event()] for k in ("x_in", "x_free", "y_ready", "y_free")}
    step_x = (lambda x: chain.run(x, [Wmine])) if world == 1 else (lambda x: stage.step(Wmine, x))

    def e2e_step(i):
        b = i & 1
        if first_rank:
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev["x_free"][b])          # the step that last read this buffer has finished
                xbufs[b].copy_(X_host, non_blocking=True)
                ev["x_in"][b].record(s_in)
            cur.wait_event(ev["x_in"][b])
        y = step_x(xbufs[b])
        if first_rank:
            ev["x_free"][b].record(cur)
        if last_rank:
            cur.wait_event(ev["y_free"][b])               # the copy-out that last used this staging buffer has finished
            ybufs[b].copy_(y, non_blocking=True)          # device to device: frees the chain's output for the next step
            ev["y_ready"][b].record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev["y_ready"][b])
                yhost[b].copy_(ybufs[b], non_blocking=True)
                ev["y_free"][b].record(s_out)

    for i in range(4):
        e2e_step(i)
    torch.cuda.synchronize(dev)
    barrier()
    a3, b3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    a3.record()
    for i in range(K_steps):
        e2e_step(i)
    cur.wait_stream(s_out)
    cur.wait_stream(s_in)
    b3.record()
    torch.cuda.synchronize(dev)
    barrier()
    e2e_ms = max_over_ranks(a3.elapsed_time(b3)) / K_steps
    checker()

    # ---- every stage's output of the last step against a library matmul of the same input on the same GPU (outside all timed
    # regions; the chain's bit-level parity with the CPU oracle is what the tests cover, this guards the timed configuration)
    last_x = xbufs[(K_steps - 1) & 1]
    if world == 1:
        inp, got = last_x, chain.Y[0]
    else:
        inp, got = (last_x if rank == 0 else stage.Yin), stage.Yout
    torch.cuda.synchronize(dev)
    barrier()
    ref = torch.matmul(inp[:1024], Wmine.t()).float()
    g1k = got[:1024].float()
    stage_rel = max_over_ranks(float((g1k - ref).abs().max() / ref.abs().max()))
    assert stage_rel <= 2e-2, f"a stage's output differs from a library matmul of its input: {stage_rel}"
    barrier()

    # ---- the last step against the CPU oracle, on the first 256 token rows (rows are independent, so a row sample is a complete
    # check of those rows): (1) every stage's output against the oracle's stage applied to the rows THAT STAGE READ on the device
    # (the tolerance of the task -- max relative error 2e-2, mean absolute error 1e-3, both after normalising by the output RMS --
    # is a per-implementation-step bound); (2) the chain's final output against the oracle run from X through ALL stages on the
    # host: asserted up to two stages (the 2-layer configuration), reported beyond, where the bf16 rounding of every
    # inter-stage activation makes two correct implementations drift apart by about 1e-3 x sqrt(stages)
    ROWS = 256
    if world == 1:
        mine = torch.stack([last_x[:ROWS], chain.Y[0][:ROWS]]).cpu()
    else:
        mine = torch.stack([(last_x if rank == 0 else stage.Yin)[:ROWS], stage.Yout[:ROWS]]).cpu()
    bits = mine.contiguous().view(torch.int32)                      # raw bits: the side group's backend has no bf16
    if world > 1:
        allbits = [torch.empty_like(bits) for _ in range(world)]
        dist.all_gather(allbits, bits, group=gloo)
    else:
        allbits = [bits]
    oracle_check = None
    if rank == 0:
        from oracle import chain as oc
        torch.set_num_threads(os.cpu_count() or 1)
        g2 = torch.Generator().manual_seed(0)
        x_rows = torch.randn(M, NK, generator=g2).to(torch.bfloat16)[:ROWS]
        assert torch.equal(x_rows, X_host[:ROWS])
        Ws_cpu = [(torch.randn(NK, NK, generator=g2) / NK ** 0.5).to(torch.bfloat16) for _ in range(n)]
        io = [b.view(torch.bfloat16) for b in allbits]             # per stage: [input rows, output rows] as the device had them
        assert torch.equal(io[0][0], x_rows)
        per_stage = [oc.error_stats(io[s][1], oc.chain_reference(io[s][0], [Ws_cpu[s]])) for s in range(n)]
        links_ok = all(torch.equal(io[s][1], io[s + 1][0]) for s in range(n - 1))     # what stage s stored is what stage s+1 read
        mx, mean = oc.error_stats(io[n - 1][1], oc.chain_reference(x_rows, Ws_cpu))
        ps_mx, ps_mean = max(p[0] for p in per_stage), max(p[1] for p in per_stage)
        ok = ps_mx <= 2e-2 and ps_mean <= 1e-3 and links_ok and (n > 2 or (mx <= 2e-2 and mean <= 1e-3))
        oracle_check = {"rows": ROWS, "stages": n, "per_stage_max_rel": ps_mx, "per_stage_mean_abs": ps_mean, "links_bit_identical": links_ok,
                        "chain_max_rel": mx, "chain_mean_abs": mean, "bounds": [2e-2, 1e-3], "ok": bool(ok)}
        del Ws_cpu
    barrier()

    # ---- the north-star records that go with the line (untimed extras): the gated single-run latency of the two-stage chain
    # against one library GEMM, and the tensor-parallel layer boundary against cuBLAS + NCCL + fused norm at TP = N
    latency = boundary = None
    if world >= 2 and not args.no_extras:
        step = step_x = checker = stage = None       # the chain's buffers go before the extras allocate theirs
        X_dev = xbufs = ybufs = inp = got = last_x = None
        torch.cuda.empty_cache()
        barrier()
        if rank == 0:
            try:
                latency = latency_record([4096, 8192], GEMM_CFG)
            except Exception as e:  # noqa: BLE001
                latency = {"error": repr(e)[:300]}
            torch.cuda.synchronize(0); torch.cuda.synchronize(1)
            torch.cuda.empty_cache()
        barrier()
        from ctapp import tp4
        tp4.GLOO = gloo
        bargs = argparse.Namespace(**{**vars(args), "shape": "B", "steps": 10, "warmup": 3, "baselines": "stock"})
        try:
            boundary = boundary_record(bargs, rank, world, dev, M=4096, with_eager=False)
        except Exception as e:  # noqa: BLE001
            boundary = {"error": repr(e)[:300]}
        barrier()

    if rank != 0:
        return
    burst, sustained, kind = peaks()
    line = {"metric": "chain_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": K_steps, "warmup": W_steps,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args, n), "clocks": clk.summary(),
            "e2e": {"value": flops_step / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": M * NK * 2, "d2h_bytes_per_step": M * NK * 2},
            "gpu_launches": launches_per_step * K_steps, "stage_output_check_max_rel": stage_rel, "oracle_check": oracle_check,
            "sustained": {"ms_per_step": sustained_ms, "value": flops_step / (sustained_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": n_tail,
                          "note": "the same steps back to back for about a second; the clocks key was sampled over the timed region plus this loop"}}
    if latency is not None:
        line["latency"] = {"what": "2-stage chain on GPUs 0 and 1, one gated run (host launch cost outside the window), median; ideal = one "
                                   "library GEMM = both layers on one GPU / 2; target over_ideal <= 1.15 at M >= 4096", "rows": latency}
    if boundary is not None:
        line["boundary"] = boundary
    assert oracle_check["ok"], f"the timed configuration's output differs from the CPU oracle: {oracle_check}"
    if True:
        ach = 2 * M * NK * NK / (kernel_ms * 1e-3) / 1e12
        line["roofline"] = {"bound": "tensor", "achieved": ach, "peak": burst, "unit": "TFLOP/s", "frac": ach / burst,
                            "traffic": dram_traffic(args.cfg, M),
                            "peak_kind": f"{kind} burst bf16 ({'kernel timed alone' if world == 1 else 'per GPU: one stage kernel spans the pipelined run'}, {kernel_ms:.3f} ms per launch)",
                            "frac_of_sustained": ach / sustained, "kernel": {10: "gemm2_kernel<false, false>", 11: "gemm2_kernel<false, true>", 3: "gemm_kernel<256>"}[args.cfg], "flop_per_launch": 2 * M * NK * NK}
    if not args.no_cpu_baseline and world == 1:
        reps = 3
        best, tf = cpu_chain_reference(min(M, 8192), 1, reps, os.cpu_count())
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": f"one stage (M={min(M, 8192)}, N=K={NK}) of the chain, best of {reps}, torch CPU fp32 F.linear, {best:.2f} s"}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
