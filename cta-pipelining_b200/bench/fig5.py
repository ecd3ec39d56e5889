"""2-layer chain on 2 GPUs, M sweep, gated latency: the CTA-pipelined chain against one GPU doing both layers (half of
which is the ideal: one GEMM's time), micro-batching with peer copies (best chunk), and tensor parallelism with an NCCL
all-reduce.  Mirrors reference bench/fig5.py:29-93.  One process drives both GPUs.  The chain is timed with the reference's
row-panel scoreboard (``--groups``) and with k-chunk dependencies (``--kchunk``); the best of all is reported as ``ctapp_us``.

    python cta-pipelining_b200/bench/fig5.py [--ms 1024,2048,4096,8192,16384,32768] [--reps 20] [--out fig5.json]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

from ctapp import methods as mt  # noqa: E402
from ctapp.timing import measure  # noqa: E402

N = K = 8192


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ms", default="1024,2048,4096,8192,16384,32768")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--cfg", type=int, default=10)
    ap.add_argument("--groups", default="1,2,4,ramp")
    ap.add_argument("--kchunk", default="10:11:4,10:11:2,10:10:4", help="k-chunk variants producer_cfg:consumer_cfg:group_rows, comma separated ('' = none): "
                    "the consumer's main loops stream behind the producer's tiles instead of waiting for whole row panels")
    ap.add_argument("--out", default=None)
    ap.add_argument("--skip-baselines", action="store_true", help="only the ideal, this library on one GPU and the pipelined chain")
    a = ap.parse_args()
    assert torch.cuda.device_count() >= 2, "needs 2 GPUs"
    g = torch.Generator().manual_seed(0)
    W1 = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    W2 = (torch.randn(N, N, generator=g) / N ** 0.5).to(torch.bfloat16)
    W1a, W2a, W2b = W1.to(mt.dev(0)), W2.to(mt.dev(0)), W2.to(mt.dev(1))
    rows = []
    for M in [int(v) for v in a.ms.split(",")]:
        X = torch.randn(M, K, generator=g).to(torch.bfloat16).to(mt.dev(0))
        r = {"M": M}
        one = mt.OneGpuCublas(M, X, W1a, W2a)
        r["one_gpu_cublas_us"] = measure(one, a.reps, devs=(0,))[0]
        r["ideal_us"] = r["one_gpu_cublas_us"] / 2
        ours1 = mt.OneGpuTma(M, X, W1a, W2a, a.cfg)
        r["one_gpu_ours_us"] = measure(ours1, a.reps, devs=(0,))[0]
        best, tp = None, None
        for chunk in (256, 512, 1024, 2048, 4096, 8192, 16384, 32768):
            if chunk > M or a.skip_baselines:
                break
            t = measure(mt.MicroBatchCublas(M, X, W1a, W2b, chunk), a.reps)[0]
            if best is None or t < best[0]:
                best = (t, chunk)
        if not a.skip_baselines:
            r["microbatch_cublas_us"], r["microbatch_chunk"] = best
            tp = mt.TensorParallel2(M, X, W1a, W2b)
            r["tp2_cublas_nccl_us"] = measure(tp, a.reps)[0]
        bestc = None
        for gr in [v if v in ("ramp", "head") else int(v) for v in a.groups.split(",")]:
            c = mt.Ctapp(M, X, W1a, W2b, a.cfg, a.cfg, gr)
            t = measure(c, a.reps)[0]
            c.pl.check()
            r[f"ctapp_g{gr}_us"] = t
            if bestc is None or t < bestc[0]:
                bestc = (t, gr)
        for var in [v for v in a.kchunk.split(",") if v]:
            c1, c2, gr = (int(x) for x in var.split(":"))
            c = mt.Ctapp(M, X, W1a, W2b, c1, c2, gr, scoreboard="kchunk")
            t = measure(c, a.reps)[0]
            c.pl.check()
            r[f"ctapp_kchunk_{var}_us"] = t
            if bestc is None or t < bestc[0]:
                bestc = (t, f"kchunk {var}")
        r["ctapp_us"], r["ctapp_group_rows"] = bestc
        r["ctapp_over_ideal"] = r["ctapp_us"] / r["ideal_us"]
        if not a.skip_baselines:
            r["reduction_vs_microbatch_pct"] = 100 * (1 - r["ctapp_us"] / r["microbatch_cublas_us"])
            r["reduction_vs_tp_pct"] = 100 * (1 - r["ctapp_us"] / r["tp2_cublas_nccl_us"])
        r["chain_tflops"] = 2 * 2 * M * N * K / (r["ctapp_us"] * 1e-6) / 1e12
        print(json.dumps({k: (round(v, 2) if isinstance(v, float) else v) for k, v in r.items()}), flush=True)
        rows.append(r)
        del one, ours1, tp, X
        torch.cuda.empty_cache()
    if a.out:
        json.dump(rows, open(a.out, "w"), indent=1)


if __name__ == "__main__":
    main()
