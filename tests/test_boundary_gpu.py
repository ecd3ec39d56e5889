"""The tensor-parallel boundary through the C ABI against the CPU oracle.

One GPU plays every rank here (``LocalGroup`` with a repeated device, phases launched in dependency order so nothing waits
on the device); with 2+ GPUs the same objects run one rank per GPU, concurrently.  Checked per case:
  * x and out against the oracle's model of the device rounding sequence (>= 99 % of the elements within one bf16 ulp, and
    max relative error <= 2e-2 / mean absolute error <= 1e-3 after normalising by the output RMS);
  * x and out against the fp32 reference within the reference's own tolerance (max|a-b| / max|b| < 1e-2 for x, < 2e-2 for out);
  * x bit-identical on all ranks; every tile flag of the owned panels and every panel flag == epoch; 128 arrivals per panel.
"""
import pytest
import torch

from oracle import boundary as ob
from oracle import chain as oc

pytestmark = pytest.mark.gpu


def rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max()).item()


def _ulp_frac(a, b):
    return ((a.view(torch.int16).int() - b.view(torch.int16).int()).abs() <= 1).float().mean().item()


def _setup(world, devices, max_M, K, n1, N2_, **kw):
    from ctapp.symm import LocalGroup
    from ctapp.tp4 import CtappBoundary
    grp = LocalGroup(devices)
    Kr, N2r = K // world, N2_ // world
    return [CtappBoundary(max_M, Kr, N2r, r, world, grp, torch.device("cuda", devices[r]), protocol="v5", max_M=max_M, n1=n1,
                          fusion="serial", **kw) for r in range(world)]


def _forward_and_check(bds, M, K, n1, N2_, seed, use_resid=True, out_ulp=0.98):
    from ctapp.tp4 import forward_lockstep
    world = len(bds)
    Kr, N2r = K // world, N2_ // world
    Wd, gamma, Wq = ob.make_weights(seed=seed, K=K, N2_=N2_, n1=n1)
    h, resid = ob.make_inputs(M, seed=seed + 100, K=K, n1=n1)
    if not use_resid:
        resid = None
    sh = [ob.shard_weights(Wd, Wq, gamma, r, world) for r in range(world)]
    devs = [bd.dev for bd in bds]
    outs = forward_lockstep(bds, [h[:, r * Kr:(r + 1) * Kr].contiguous().to(devs[r]) for r in range(world)],
                            [resid.to(devs[r]) if resid is not None else None for r in range(world)],
                            [sh[r][0].to(devs[r]) for r in range(world)], [sh[r][2].to(devs[r]) for r in range(world)])
    for bd in bds:
        bd.check()
    x_model, out_model = ob.boundary_device_model(h, Wd, resid, gamma, Wq, world)
    x_ref, out_ref = ob.boundary_reference(h, Wd, resid, gamma, Wq)
    xs = [bd.x().cpu() for bd in bds]
    for r in range(world):
        assert torch.equal(xs[r], xs[0]), f"x differs between rank {r} and rank 0"
    assert _ulp_frac(xs[0], x_model) >= 0.99, _ulp_frac(xs[0], x_model)
    mx, mean = oc.error_stats(xs[0], x_model)
    assert mx <= 2e-2 and mean <= 1e-3, ("x vs model", mx, mean)
    assert rel(xs[0], x_ref) < 1e-2, rel(xs[0], x_ref)
    out = torch.cat([o.cpu() for o in outs], dim=1)
    assert not torch.isnan(out.float()).any()
    mx, mean = oc.error_stats(out, out_model)
    assert mx <= 2e-2 and mean <= 1e-3, ("out vs model", mx, mean)
    assert _ulp_frac(out, out_model) >= out_ulp, _ulp_frac(out, out_model)
    assert rel(out, out_ref) < 2e-2, rel(out, out_ref)
    # protocol state
    P = M // 128
    for r, bd in enumerate(bds):
        Pr = ob.panels_owned(M, r, world)
        assert (bd.tile_flags[:, :Pr, :].cpu() == bd.epoch).all(), f"rank {r}: a tile flag of an owned panel != epoch {bd.epoch}"
        assert (bd.panel_flag[:P].cpu() == bd.epoch).all(), f"rank {r}: a panel flag != epoch {bd.epoch}"
        own = [m for m in range(P) if m % world == r]
        assert (bd.panel_done[own].cpu() == (n1 // 256) * 4).all()
        assert int(bd.epoch_dev.item()) == bd.epoch


@pytest.mark.parametrize("cta_pair,kw", [(True, {}), (True, dict(steal=True)), (False, dict(down_raster=2)), (False, dict(steal=True, down_tail=0)),
                                         ("wide", {}), ("wide", dict(down_tail=1))])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_boundary_one_gpu_plays_all_ranks(world, cta_pair, kw):
    """``steal`` here: the dedicated reducers claim their units from the shared counter and the mode-8 consumers, launched after
    them, find it exhausted; ``down_raster=2``: producer and reducer walk panel by panel."""
    K, n1, N2_ = 1024 * world if world < 8 else 2048, 512, 256 * world
    bds = _setup(world, [0] * world, 1024, K, n1, N2_, cta_pair=cta_pair, **kw)
    for seed, M in enumerate((1024, 256, 640, 128), start=3):   # variable M on one instance, fresh weights per call
        _forward_and_check(bds, M, K, n1, N2_, seed)


def test_boundary_no_residual_and_tile128():
    bds = _setup(2, [0, 0], 512, 512, 768, 512, resid=False, qkv_tile=128, down_tail=0)
    _forward_and_check(bds, 512, 512, 768, 512, 11, use_resid=False)
    _forward_and_check(bds, 384, 512, 768, 512, 12, use_resid=False)


@pytest.mark.parametrize("cta_pair", [True, False])
def test_consumer_ctas_do_the_whole_reduction(cta_pair):
    """``steal`` with no dedicated reducer CTAs (R = 0): every unit is claimed and reduced by warps of the consumer GEMM's CTAs
    before they start on their tiles (one rank; with more ranks on one GPU a consumer would wait for panels whose owners'
    consumers have not been launched yet)."""
    bds = _setup(1, [0], 1024, 1024, 1024, 768, cta_pair=cta_pair, steal=True, R=0)
    for seed, M in enumerate((1024, 384, 1024), start=40):
        _forward_and_check(bds, M, 1024, 1024, 768, seed)
        assert int(bds[0].role_ctr[1].item()) >= (M // 128) * (1024 // 256) * 4      # every unit was claimed from the counter


def test_boundary_headline_shape_vs_oracle():
    """The benchmarked boundary shape -- M = 4096 tokens, down-projection K = 28672 (two ranks of 14336), hidden 8192, QKV width
    10240 -- with one GPU playing both ranks, against the CPU oracle (about 5 TFLOP on the host cores)."""
    bds = _setup(2, [0, 0], 4096, 28672, 8192, 10240)
    # x is one bf16 rounding of an fp32 sum either way; out inherits x's rare one-ulp differences through an 8192-long dot
    # product and a scale, so a few more of its elements land on the neighbouring bf16 than in the small cases
    _forward_and_check(bds, 4096, 28672, 8192, 10240, 77, out_ulp=0.97)


def test_thirty_forwards_alternating_shapes_and_inputs():
    """Back-to-back stress (reference tests/test_tp4.py:216-263): 30 forwards on one instance without a host synchronisation
    in between, alternating (M, inputs, weights); every output and x is cloned on the stream and checked afterwards."""
    from ctapp.symm import LocalGroup
    from ctapp.tp4 import CtappBoundary
    K, n1, N2_, max_M = 512, 1024, 512, 1024
    bd = CtappBoundary(max_M, K, N2_, 0, 1, LocalGroup([0]), torch.device("cuda", 0), protocol="v5", n1=n1, fusion="serial")
    cases = []
    for i, M in enumerate((1024, 256, 768, 128)):
        Wd, gamma, Wq = ob.make_weights(seed=80 + i, K=K, N2_=N2_, n1=n1)
        h, resid = ob.make_inputs(M, seed=90 + i, K=K, n1=n1)
        wd, _, wqf = ob.shard_weights(Wd, Wq, gamma, 0, 1)
        cases.append((h.cuda(), resid.cuda(), wd.cuda(), wqf.cuda(), ob.boundary_device_model(h, Wd, resid, gamma, Wq, 1)))
    got = []
    for it in range(30):
        h, resid, wd, wqf, _ = cases[(it * 3 + it // 4) % 4]
        out = bd.forward(h, resid, wd, wqf)
        got.append((out.clone(), bd.x().clone()))
    bd.check()
    for it, (out, x) in enumerate(got):
        x_model, out_model = cases[(it * 3 + it // 4) % 4][4]
        assert _ulp_frac(x.cpu(), x_model) >= 0.99 and _ulp_frac(out.cpu(), out_model) >= 0.98, it
    assert bd.epoch == 30 and int(bd.epoch_dev.item()) == 30


def test_fifty_forwards_cycling_M_eager_and_graphs():
    """Soak (reference tests/test_tp4.py:266-300): 50 forwards cycling the token count, eager and with one CUDA graph per
    (parity, M); the last output of every M is checked and the device epoch must have followed the host's."""
    from ctapp.symm import LocalGroup
    from ctapp.tp4 import CtappBoundary
    K, n1, N2_, max_M = 512, 512, 512, 1024
    Wd, gamma, Wq = ob.make_weights(seed=7, K=K, N2_=N2_, n1=n1)
    wd, _, wqf = ob.shard_weights(Wd, Wq, gamma, 0, 1)
    Ms = (1024, 512, 256, 768, 128)
    data = {M: ob.make_inputs(M, seed=M, K=K, n1=n1) for M in Ms}
    model = {M: ob.boundary_device_model(data[M][0], Wd, data[M][1], gamma, Wq, 1) for M in Ms}
    for use_graph in (False, True):
        bd = CtappBoundary(max_M, K, N2_, 0, 1, LocalGroup([0]), torch.device("cuda", 0), protocol="v5", n1=n1, fusion="serial", use_graph=use_graph)
        bd.set_weights(wd.cuda(), wqf.cuda())
        last = {}
        for it in range(50):
            M = Ms[it % len(Ms)] if it % 7 else Ms[(it // 7) % len(Ms)]
            out = bd.forward(data[M][0].cuda(), data[M][1].cuda())
            last[M] = (out.clone(), bd.x().clone())
        bd.check()
        assert int(bd.epoch_dev.item()) == bd.epoch == 50
        if use_graph:
            assert 2 <= len(bd._graphs.graphs) <= 2 * len(Ms)      # one graph per (parity, M) seen after the first, eager, forward
        for M, (out, x) in last.items():
            assert _ulp_frac(x.cpu(), model[M][0]) >= 0.99 and _ulp_frac(out.cpu(), model[M][1]) >= 0.98, (use_graph, M)


def test_boundary_hidden_8192_one_rank_vs_oracle():
    """The real hidden size (8192) with a reduced K so the CPU oracle finishes in seconds."""
    bds = _setup(1, [0], 512, 1024, 8192, 1280)
    _forward_and_check(bds, 512, 1024, 8192, 1280, 21)


def test_boundary_single_rank_public_forward_and_floor():
    """world 1 through the public ``forward`` (serial fusion), eager and CUDA graph, plus the protocol-free floor."""
    from ctapp.symm import LocalGroup
    from ctapp.tp4 import CtappBoundary
    M, K, n1, N2_ = 256, 512, 512, 512
    Wd, gamma, Wq = ob.make_weights(seed=5, K=K, N2_=N2_, n1=n1)
    h, resid = ob.make_inputs(M, seed=6, K=K, n1=n1)
    wd, _, wqf = ob.shard_weights(Wd, Wq, gamma, 0, 1)
    x_model, out_model = ob.boundary_device_model(h, Wd, resid, gamma, Wq, 1)
    for use_graph in (False, True):
        bd = CtappBoundary(M, K, N2_, 0, 1, LocalGroup([0]), torch.device("cuda", 0), protocol="v5", n1=n1, fusion="serial", use_graph=use_graph)
        bd.set_weights(wd.cuda(), wqf.cuda())
        for i in range(5):
            out = bd.forward(h.cuda(), resid.cuda())
            bd.check()
            assert _ulp_frac(out.cpu(), out_model) >= 0.98 and _ulp_frac(bd.x().cpu(), x_model) >= 0.99, (use_graph, i)
    fl = CtappBoundary(M, K, N2_, 0, 1, LocalGroup([0]), torch.device("cuda", 0), protocol=False, n1=n1)
    y = fl.forward(h.cuda(), None, wd.cuda(), wqf.cuda())
    torch.cuda.synchronize()
    ref = ((h.float() @ wd.float().t()).to(torch.bfloat16).float() @ wqf.float().t()).to(torch.bfloat16)
    assert _ulp_frac(y.cpu(), ref) >= 0.98


def test_reducer_missing_producer_times_out_cleanly():
    """Fault injection on the host: the owner reducer is launched although no producer will raise its tile flags.  Its
    bounded wait must give up with code 3 and leave the context usable."""
    from ctapp.ext import load_tp4
    ext = load_tp4()
    ext.set_wait_limit_ms(50)
    try:
        bds = _setup(1, [0], 256, 256, 512, 256)
        bd = bds[0]
        bd.epoch += 1
        bd._step(256)
        bd.launch_reducer(256, None, 1)
        torch.cuda.synchronize()
        s = bd.status.cpu().tolist()
        assert s[0] == 3 and s[3] == 1, s
        with pytest.raises(RuntimeError):
            bd.check()
        _forward_and_check(_setup(1, [0], 256, 256, 512, 256), 256, 256, 512, 256, 31)
    finally:
        ext.set_wait_limit_ms(2000)


def test_add_rmsnorm_baseline_kernel():
    from ctapp.ext import load_tp4
    from ctapp.tp4 import rmsnorm_gamma
    ext = load_tp4()
    g = torch.Generator().manual_seed(0)
    a = torch.randn(64, 8192, generator=g).to(torch.bfloat16).cuda(); r = torch.randn(64, 8192, generator=g).to(torch.bfloat16).cuda()
    gamma = (0.5 + torch.rand(8192, generator=g)).to(torch.bfloat16).cuda()
    x, y = torch.empty_like(a), torch.empty_like(a)
    ext.add_rmsnorm(a, r, gamma, x, y)
    torch.cuda.synchronize()
    xr = a + r
    assert torch.equal(x, xr)
    assert _ulp_frac(y, rmsnorm_gamma(xr, gamma)) >= 0.99


@pytest.mark.multigpu(2)
@pytest.mark.parametrize("cta_pair,kw", [(True, {}), (False, {}), (True, dict(steal=True)), (True, dict(steal=True, R=0)), (False, dict(steal=True)),
                                         (True, dict(R=0, red_blocks=48, red_threads=256))])     # last: reducer CTAs share SMs with the GEMMs' CTAs
@pytest.mark.parametrize("world,fusion", [(2, "none"), (2, "pdl"), (2, "pdl1")])
def test_boundary_two_gpus_concurrent(world, fusion, cta_pair, kw):
    """One rank per GPU, driven from this process: producer || reducer || consumer overlap within and across GPUs."""
    _concurrent_case(world, fusion, cta_pair, kw)


@pytest.mark.multigpu(2)
@pytest.mark.parametrize("cta_pair,kw", [(True, {}), (True, dict(R=8)), (False, dict(R=6)), (True, dict(steal=True)), (True, dict(steal=True, R=0)),
                                         (False, dict(steal=True))])
def test_boundary_two_gpus_role_switching(cta_pair, kw):
    """fusion="role": no reducer kernel; the first R consumer CTAs to arrive run the reducer's static shares (with steal: every
    consumer CTA claims units), then take GEMM tiles.  Same results as every other variant."""
    _concurrent_case(2, "role", cta_pair, kw)


def _concurrent_case(world, fusion, cta_pair, kw):
    from ctapp.symm import LocalGroup
    from ctapp.tp4 import CtappBoundary
    K, n1, N2_, max_M = 4096, 8192, 2560, 2048
    grp = LocalGroup(list(range(world)))
    Kr, N2r = K // world, N2_ // world
    bds = [CtappBoundary(max_M, Kr, N2r, r, world, grp, torch.device("cuda", r), protocol="v5", max_M=max_M, n1=n1, fusion=fusion, cta_pair=cta_pair, **kw) for r in range(world)]
    Wd, gamma, Wq = ob.make_weights(seed=1, K=K, N2_=N2_, n1=n1)
    sh = [ob.shard_weights(Wd, Wq, gamma, r, world) for r in range(world)]
    wds = [sh[r][0].to(bds[r].dev) for r in range(world)]; wqs = [sh[r][2].to(bds[r].dev) for r in range(world)]
    for it, M in enumerate((2048, 512, 1024, 2048, 2048)):
        h, resid = ob.make_inputs(M, seed=40 + it, K=K, n1=n1)
        outs = [bds[r].forward(h[:, r * Kr:(r + 1) * Kr].contiguous().to(bds[r].dev), resid.to(bds[r].dev), wds[r], wqs[r]) for r in range(world)]
        for bd in bds:
            bd.check()
        x_model, out_model = ob.boundary_device_model(h, Wd, resid, gamma, Wq, world)
        xs = [bd.x().cpu() for bd in bds]
        assert all(torch.equal(x, xs[0]) for x in xs)
        assert _ulp_frac(xs[0], x_model) >= 0.99
        out = torch.cat([o.cpu() for o in outs], dim=1)
        assert _ulp_frac(out, out_model) >= 0.98
        mx, mean = oc.error_stats(out, out_model)
        assert mx <= 2e-2 and mean <= 1e-3


def test_boundary_pool_one_instance_serves_every_supported_M():
    """``CtappBoundaryPool`` (reference tests/test_tp4_pool.py:17-83): unsupported token counts give None (the caller keeps its
    stock path), every supported one is served by the same instance with the weights of the call."""
    from ctapp.symm import LocalGroup
    from ctapp.tp4 import CtappBoundaryPool
    K, n1, N2_ = 512, 512, 512
    pool = CtappBoundaryPool(K, N2_, 0, 1, LocalGroup([0]), torch.device("cuda", 0), min_M=256, max_M=1024, n1=n1, fusion="serial")
    assert pool.get(200) is None and pool.get(128) is None and pool.get(2048) is None and pool.get(1000) is None
    seen = set()
    for i, M in enumerate((512, 1024, 256, 768, 512)):
        bd = pool.get(M)
        seen.add(id(bd))
        Wd, gamma, Wq = ob.make_weights(seed=60 + i, K=K, N2_=N2_, n1=n1)
        h, resid = ob.make_inputs(M, seed=70 + i, K=K, n1=n1)
        wd, _, wqf = ob.shard_weights(Wd, Wq, gamma, 0, 1)
        out = bd.forward(h.cuda(), resid.cuda(), wd.cuda(), wqf.cuda())
        bd.check()
        x_model, out_model = ob.boundary_device_model(h, Wd, resid, gamma, Wq, 1)
        assert out.shape == (M, N2_) and bd.x().shape == (M, n1)
        assert _ulp_frac(bd.x().cpu(), x_model) >= 0.99 and _ulp_frac(out.cpu(), out_model) >= 0.98, (i, M)
    assert len(seen) == 1 and len(pool._inst) == 1


def test_silu_mul_kernel_vs_oracle():
    from ctapp.ext import load_tp4
    ext = load_tp4()
    g = (torch.randn(300, 2000, generator=torch.Generator().manual_seed(3)) * 2).to(torch.bfloat16)
    out = ext.silu_mul(g.cuda())
    torch.cuda.synchronize()
    ref = ob.silu_and_mul(g)
    d = (out.cpu().view(torch.int16).int() - ref.view(torch.int16).int()).abs()
    assert int(d.max()) <= 1 and (d == 0).float().mean().item() >= 0.995, (int(d.max()), (d == 0).float().mean().item())


@pytest.mark.parametrize("M,K,I", [(512, 1024, 512), (384, 512, 1280), (4096, 1024, 1792)])
def test_consumer_gemm_activation_epilogue(M, K, I):
    """silu(gate) * up fused into the consumer GEMM's epilogue (weight rows interleaved in blocks of 128) against the same
    kernel without the fusion followed by the oracle's activation (at most one bf16 ulp apart: same accumulators, same
    rounding before the activation) and against the fp32 reference within the boundary's tolerance."""
    from ctapp.ext import load_tp4
    from ctapp.tp4 import interleave_gate_up
    ext = load_tp4()
    g = torch.Generator().manual_seed(11)
    X = torch.randn(M, K, generator=g).to(torch.bfloat16)
    W = (torch.randn(2 * I, K, generator=g) / K ** 0.5 * 2).to(torch.bfloat16)        # rows: gate, then up
    rowss = (torch.rand(M, generator=g) + 0.5) * K
    Wi = interleave_gate_up(W)
    assert torch.equal(Wi[:128], W[:128]) and torch.equal(Wi[128:256], W[I:I + 128]) and torch.equal(Wi[256:384], W[128:256])
    Xd, Wd_, Wid, rs = X.cuda(), W.cuda(), Wi.cuda(), rowss.cuda()
    plain = torch.empty(M, 2 * I, dtype=torch.bfloat16, device="cuda")
    fused = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device="cuda")
    ext.tp4_qkv(Xd, Wd_, plain, 2, 1, 0, 0, rowss=rs, cta_pair=1)
    ext.tp4_qkv(Xd, Wid, fused, 2, 1, 0, 0, rowss=rs, cta_pair=1, act=1)
    torch.cuda.synchronize()
    want = ob.silu_and_mul(plain.cpu())
    d = (fused.cpu().view(torch.int16).int() - want.view(torch.int16).int()).abs()
    assert int(d.max()) <= 1 and (d == 0).float().mean().item() >= 0.99, (int(d.max()), (d == 0).float().mean().item())
    out32 = (X.float() @ W.float().t()) * torch.rsqrt(rowss / K + 1e-5)[:, None]
    ref = ob.silu_and_mul(out32.to(torch.bfloat16))
    mx, mean = oc.error_stats(fused.cpu(), ref)
    assert mx <= 2e-2 and mean <= 1e-3, (mx, mean)
    with pytest.raises(RuntimeError):
        ext.tp4_qkv(Xd, Wid, fused, 2, 1, 0, 0, rowss=rs, cta_pair=0, act=1)          # the one-CTA kernel has no such epilogue


@pytest.mark.parametrize("world", [1, 2])
def test_boundary_with_activation_epilogue(world):
    """The whole boundary with a gate/up consumer: every rank's out is silu(gate_r) * up_r of the oracle's model output."""
    from ctapp.tp4 import forward_lockstep, interleave_gate_up
    M, K, n1, N2_ = 512, 1024, 2048, 2048
    bds = _setup(world, [0] * world, M, K, n1, N2_, act=True)
    Kr, N2r = K // world, N2_ // world
    Wd, gamma, Wq = ob.make_weights(seed=5, K=K, N2_=N2_, n1=n1)
    h, resid = ob.make_inputs(M, seed=105, K=K, n1=n1)
    sh = [ob.shard_weights(Wd, Wq, gamma, r, world) for r in range(world)]
    outs = forward_lockstep(bds, [h[:, r * Kr:(r + 1) * Kr].contiguous().cuda() for r in range(world)], [resid.cuda()] * world,
                            [sh[r][0].cuda() for r in range(world)], [interleave_gate_up(sh[r][2]).cuda() for r in range(world)])
    for bd in bds:
        bd.check()
    _, out_model = ob.boundary_device_model(h, Wd, resid, gamma, Wq, world)
    for r in range(world):
        assert tuple(outs[r].shape) == (M, N2r // 2)
        want = ob.silu_and_mul(out_model[:, r * N2r:(r + 1) * N2r].contiguous())
        mx, mean = oc.error_stats(outs[r].cpu(), want)
        assert mx <= 2e-2 and mean <= 1e-3, (r, mx, mean)
        assert _ulp_frac(outs[r].cpu(), want) >= 0.97, _ulp_frac(outs[r].cpu(), want)
