"""Per-rank bodies of the multi-process GPU tests (one process per GPU, spawned through ``ctapp.tp4.launch``).  Each returns
a list of failure strings (empty = pass)."""
import torch
import torch.distributed as dist


def _sync(dev):
    from ctapp import tp4
    torch.cuda.synchronize(dev)
    tp4.barrier()


def nvls_probes(rank, world, dev, gn):
    """Known answers for the multimem operations the NVLS variant uses (reference tests/test_tp4.py:44-107)."""
    from ctapp.ext import load_tp4
    from ctapp.symm import symm_empty
    ext = load_tp4()
    fails = []
    buf, h = symm_empty((4096,), torch.int32, dev, gn, rank, multicast=True)
    if not h.multicast_ptr:
        return ["SKIP: no multicast address on this system"]
    for n in (1, 100, 4096):
        buf.zero_(); _sync(dev)
        ext.mm_red_u32(h.multicast_ptr, n, 3); _sync(dev)
        b = buf.cpu()
        if not (bool((b[:n] == 3 * world).all()) and bool((b[n:] == 0).all())):
            fails.append(f"mm_red_u32 n={n}")
    n = 8192
    fb, fh = symm_empty((n,), torch.float32, dev, gn, rank, multicast=True)
    srcs = [torch.randn(n, generator=torch.Generator().manual_seed(100 + r)) for r in range(world)]
    fb.zero_(); _sync(dev)
    ext.mm_red_f32(fh.multicast_ptr, srcs[rank].to(dev)); _sync(dev)
    if (fb.cpu() - sum(srcs)).abs().max().item() >= 1e-4:
        fails.append("mm_red_f32")
    bb, bh = symm_empty((n,), torch.bfloat16, dev, gn, rank, multicast=True)
    bb.zero_(); _sync(dev)
    src = torch.randn(n, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16)
    if rank == 0:
        ext.mm_st_bf16(bh.multicast_ptr, src.to(dev))
    _sync(dev)
    if not torch.equal(bb.cpu(), src):
        fails.append("mm_st_bf16 broadcast")
    n = 65536
    lb, lh = symm_empty((n,), torch.bfloat16, dev, gn, rank, multicast=True)
    datas = [(torch.randn(n, generator=torch.Generator().manual_seed(200 + r)) * 0.1).to(torch.bfloat16) for r in range(world)]
    lb.copy_(datas[rank]); _sync(dev)
    out = torch.empty(n, dtype=torch.bfloat16, device=dev)
    ext.mm_ld_reduce_bf16(lh.multicast_ptr, out); _sync(dev)
    # the in-switch sum is accumulated in fp32 (proved below with 3+ ranks) but its final conversion to bf16 is not round to
    # nearest even on this hardware: about one result in five is the neighbouring bf16.  One ulp is the contract checked here
    # (the boundary itself never uses ld_reduce: the owner reducer adds in registers and rounds once, to nearest even).
    exp = sum(d.float() for d in datas).to(torch.bfloat16)
    d_ulp = (out.cpu().view(torch.int16).int() - exp.view(torch.int16).int()).abs()
    if int(d_ulp.max()) > 1:
        fails.append(f"mm_ld_reduce_bf16: off by {int(d_ulp.max())} ulp ({int((d_ulp > 1).sum())} of {n} beyond one)")
    if world >= 3:      # 256 + 1 + 1 (+...) only survives when the switch accumulates in fp32
        vals = [256.0] + [1.0] * (world - 1)
        lb.fill_(vals[rank]); _sync(dev)
        ext.mm_ld_reduce_bf16(lh.multicast_ptr, out); _sync(dev)
        # sequential bf16 accumulation would stay at 256 (256 + 1 rounds back to 256); an fp32 accumulator holds 256 + (world - 1)
        # and only the final conversion decides between the two neighbouring bf16 values
        got = out.cpu().float()
        exact = float(sum(vals))
        if not (bool((got > 256.0).all()) and bool(((got - exact).abs() <= 2.0).all())):
            fails.append(f"mm_ld_reduce_bf16 does not accumulate in fp32: got {got[0].item()} for {exact}")
    slots, iters = 64, 500
    db, dh = symm_empty((slots * 32 * 8,), torch.bfloat16, dev, gn, rank, multicast=True)
    fl, fh2 = symm_empty((slots,), torch.int32, dev, gn, rank, multicast=True)
    ak, ah = symm_empty((slots,), torch.int32, dev, gn, rank, multicast=True)
    db.zero_(); fl.zero_(); ak.zero_(); _sync(dev)
    stale, gave_up = ext.mm_order_stress(dh.multicast_ptr, db, fh2.multicast_ptr, fl, ah.multicast_ptr, ak, rank, world, iters, slots)
    _sync(dev)
    if stale or gave_up:
        fails.append(f"mm_order_stress: {stale} stale words, gave_up={gave_up}")
    return fails


def boundary_case(rank, world, dev, gn, protocol, fusion, cta_pair, Ms, K, n1, N2_, steal=False):
    """The boundary with one process per GPU against the CPU oracle; also x identical on every rank and flags == epoch."""
    import sys, os
    from ctapp import tp4
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if root not in sys.path:
        sys.path.insert(0, root)
    from oracle import boundary as ob
    from oracle import chain as oc
    fails = []
    Kr, N2r = K // world, N2_ // world
    max_M = max(Ms)
    bd = tp4.CtappBoundary(max_M, Kr, N2r, rank, world, gn, dev, protocol=protocol, max_M=max_M, n1=n1, fusion=fusion, cta_pair=cta_pair, steal=steal)
    if protocol in ("v3", "v3r") and not bd.nvls:
        return ["SKIP: no multicast address on this system"]
    # in-switch reduction: the switch returns the partials' sum as bf16 and the residual is added after that rounding: one bf16
    # rounding more than the model (and the inbox path), which adds everything in fp32 and rounds once.  x stays inside the bounds
    # (measured max 1.7e-2, mean 9.2e-4 of the RMS) but sits up to two bf16 steps from the model; out's mean error was measured
    # at 1.9e-3 of the RMS, twice the 1e-3 the other protocols are held to against this model.  The variant is opt-in for that
    # reason; this test pins what it does deliver (max 2e-2, mean 2.5e-3).
    x_ulp, out_ulp, steps, out_mean = (0.99, 0.98, 1, 1e-3) if protocol != "v3r" else (0.95, 0.85, 2, 2.5e-3)
    for it, M in enumerate(Ms):
        Wd, gamma, Wq = ob.make_weights(seed=1 + it, K=K, N2_=N2_, n1=n1)
        wd, _, wqf = ob.shard_weights(Wd, Wq, gamma, rank, world)
        h, resid = ob.make_inputs(M, seed=40 + it, K=K, n1=n1)
        out = bd.forward(h[:, rank * Kr:(rank + 1) * Kr].contiguous().to(dev), resid.to(dev), wd.to(dev), wqf.to(dev))
        bd.check()
        x_model, out_model = ob.boundary_device_model(h, Wd, resid, gamma, Wq, world)
        x = bd.x().cpu()
        ulp = lambda a, b: ((a.view(torch.int16).int() - b.view(torch.int16).int()).abs() <= steps).float().mean().item()  # noqa: E731
        mxx, meanx = oc.error_stats(x, x_model)
        if ulp(x, x_model) < x_ulp or not (mxx <= 2e-2 and meanx <= 1e-3):
            fails.append(f"M={M}: x within {steps} ulp only {ulp(x, x_model):.4f}, max {mxx:.3e} mean {meanx:.3e}")
        o = out.cpu()
        om = out_model[:, rank * N2r:(rank + 1) * N2r]
        mx, mean = oc.error_stats(o, om)
        if not (mx <= 2e-2 and mean <= out_mean and ulp(o, om) >= out_ulp):
            fails.append(f"M={M}: out max {mx:.3e} mean {mean:.3e} ulp {ulp(o, om):.4f}")
        bits = [None] * world
        dist.all_gather_object(bits, int(x.view(torch.int16).to(torch.int64).sum().item()), group=tp4.GLOO)
        if len(set(bits)) != 1:
            fails.append(f"M={M}: x differs between ranks")
        P = M // 128
        Pr = ob.panels_owned(M, rank, world)
        if not bool((bd.tile_flags[:, :Pr, :].cpu() == bd.epoch).all()) or not bool((bd.panel_flag[:P].cpu() == bd.epoch).all()):
            fails.append(f"M={M}: flags != epoch {bd.epoch}")
        _sync(dev)
    return fails


def chain_stages_case(rank, world, dev, gn, M, NK, steps, cfg, group_rows=2, scoreboard="rowpanel"):
    """One chain stage per process, ``steps`` steps enqueued back to back with a different input each and no host
    synchronisation in between: consecutive steps overlap on the doubled links, and every step's output at the last stage
    must still be the CPU oracle's chain of that step's input."""
    import sys, os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if root not in sys.path:
        sys.path.insert(0, root)
    from oracle import chain as oc
    from ctapp.pipeline import ChainStage
    fails = []
    Xs, Ws = [], None
    for e in range(steps):
        X, Ws_e = oc.make_chain_inputs(M, NK, [NK] * world, seed=e)
        Xs.append(X)
        Ws = Ws or Ws_e
    stage = ChainStage(M, NK, [NK] * world, rank, world, dev, group=None, cfg=cfg, group_rows=group_rows, scoreboard=scoreboard)
    Wmine = Ws[rank].to(dev)
    Xd = [x.to(dev) for x in Xs] if rank == 0 else [None] * steps
    outs = []
    for e in range(steps):
        y = stage.step(Wmine, Xd[e])
        if rank == world - 1:
            outs.append(y.clone())      # stream order: after this step's kernel, before the next one overwrites the output
    stage.check()
    _sync(dev)
    if rank == world - 1:
        for e in range(steps):
            ref = oc.chain_reference(Xs[e], Ws)
            mx, mean = oc.error_stats(outs[e].cpu(), ref)
            if not (mx <= 2e-2 and mean <= 1e-3):
                fails.append(f"step {e}: max {mx:.3e} mean {mean:.3e}")
    if stage.epoch != steps:
        fails.append(f"epoch {stage.epoch} != {steps}")
    if scoreboard == "kchunk" and rank > 0:      # every flag of either set carries the number of the last step that used the set
        want = [steps - 1 if (steps - 1) & 1 == s else steps for s in (0, 1)]
        got = [(int(stage.chunk2[s].min().item()), int(stage.chunk2[s].max().item())) for s in (0, 1)]
        if got != [(w, w) for w in want]:
            fails.append(f"k-chunk flags {got}, expected {want} everywhere")
    return fails
