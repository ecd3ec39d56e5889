"""Generate the golden fixtures of this directory from the Python reference.

Run once in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own pure-torch functions (ctapp.pipeline.build_deps, ctapp.tp4.shard_weights /
fold_gamma / one_gpu_reference / rmsnorm_gamma), runs them on small seeded inputs and stores inputs and
outputs as .npz.  The test-suite compares the oracle against these files; nothing reads the reference
checkout at test time.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (M, N1, N2, BM1, BN1, BM2, BN2, rowpanel)
DEPS_CASES = [
    (1024, 8192, 8192, 128, 128, 128, 128, True),     # the 2-rank chain config, 128x128 tiles
    (1024, 8192, 8192, 128, 256, 128, 256, True),     # same with 128x256 tiles
    (1024, 8192, 8192, 128, 256, 128, 256, False),
    (4096, 8192, 8192, 64, 256, 64, 256, True),
    (4096, 8192, 8192, 128, 128, 64, 256, True),      # BM1 != BM2: one producer tile feeds two panels
    (4096, 8192, 8192, 64, 256, 128, 128, True),      # BM1 < BM2: two producer rows per panel
    (4096, 8192, 10240, 128, 128, 64, 256, False),
    (1000, 1000, 520, 128, 128, 64, 256, True),       # ragged M and N
    (1000, 1000, 520, 64, 256, 128, 128, False),
    (384, 512, 768, 128, 256, 128, 256, True),
    (128, 256, 256, 128, 256, 128, 256, True),        # a single tile
    (130, 300, 300, 128, 128, 128, 128, False),       # last row panel holds 2 rows
]


def bits(t):
    """bf16 tensor -> uint16 numpy (npz has no bf16)."""
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main(ref_root):
    sys.path.insert(0, ref_root)
    from ctapp.pipeline import build_deps
    from ctapp import tp4

    out = {}
    for i, c in enumerate(DEPS_CASES):
        off, cons, init = build_deps(*c)
        out[f"case{i}_args"] = np.asarray([int(v) for v in c], dtype=np.int64)
        out[f"case{i}_off"] = off.numpy()
        out[f"case{i}_cons"] = cons.numpy()
        out[f"case{i}_init"] = init.numpy()
    # grouped producer order (ctapp/pipeline.py:48-51 is inline code in Pipeline.__init__, which needs GPUs; this is the
    # same expression evaluated on the CPU)
    for j, (P, tn1, g) in enumerate([(512, 64, 8), (256, 32, 8), (96, 32, 2), (160, 32, 4), (64, 64, 8)]):
        t = torch.arange(P); m, n = t // tn1, t % tn1
        order = torch.argsort(((m // g) * tn1 + n) * g + m % g)
        out[f"order{j}_args"] = np.asarray([P, tn1, g], dtype=np.int64)
        out[f"order{j}"] = order.numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "chain_deps.npz"), **out)

    # boundary arithmetic on small shapes (none of the reference functions used here depends on the hidden size
    # constant, so the hidden size shrinks too and the fixture stays below 1 MB)
    b = {}
    for k, (M, K, H, N2_, world, seed) in enumerate([(64, 256, 256, 192, 2, 3), (96, 512, 384, 256, 4, 4)]):
        g = torch.Generator().manual_seed(seed)
        h = torch.randn(M, K, generator=g).to(torch.bfloat16)
        resid = torch.randn(M, H, generator=g).to(torch.bfloat16)
        Wd = (torch.randn(H, K, generator=g) * K ** -0.5).to(torch.bfloat16)
        gamma = (0.5 + torch.rand(H, generator=g)).to(torch.bfloat16)
        Wq = (torch.randn(N2_, H, generator=g) * H ** -0.5).to(torch.bfloat16)
        x, o = tp4.one_gpu_reference(h, Wd, resid, gamma, Wq)
        x_nr, o_nr = tp4.one_gpu_reference(h, Wd, None, gamma, Wq)
        b[f"b{k}_args"] = np.asarray([M, K, H, N2_, world, seed], dtype=np.int64)
        for name, t in (("h", h), ("resid", resid), ("Wd", Wd), ("gamma", gamma), ("Wq", Wq)):
            b[f"b{k}_{name}"] = bits(t)
        b[f"b{k}_x"] = x.numpy(); b[f"b{k}_out"] = o.numpy()
        b[f"b{k}_x_noresid"] = x_nr.numpy(); b[f"b{k}_out_noresid"] = o_nr.numpy()
        b[f"b{k}_fold"] = bits(tp4.fold_gamma(Wq, gamma))
        b[f"b{k}_rmsnorm"] = bits(tp4.rmsnorm_gamma(x.to(torch.bfloat16), gamma))
        for r in range(world):
            wd_r, wq_r, wqf_r = tp4.shard_weights(Wd, Wq, gamma, r, world)
            b[f"b{k}_r{r}_Wd"] = bits(wd_r); b[f"b{k}_r{r}_Wq"] = bits(wq_r); b[f"b{k}_r{r}_Wqf"] = bits(wqf_r)
    np.savez_compressed(os.path.join(HERE, "boundary_small.npz"), **b)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/reference")
    main(sys.argv[1])
