"""The chain protocol on one GPU (both stages on the same device, one after the other on one stream) and, when two GPUs are
present, as a real producer/consumer pair.  Values are checked against the CPU oracle; queue order and scoreboard counts are
checked bit-exactly: against the sequential protocol model when the producer runs as a single CTA (its publish order is then
deterministic), and through order-independent invariants under full concurrency."""
import numpy as np
import pytest
import torch

from oracle import chain as oc

pytestmark = pytest.mark.gpu


def _run_case(M, K, N1, N2, cfg1, cfg2, devA, devB, runs=3, **kw):
    from ctapp.pipeline import Pipeline
    pl = Pipeline(M, K, N1, N2, cfg1, cfg2, devA=devA, devB=devB, **kw)
    X, (W1, W2) = oc.make_chain_inputs(M, K, [N1, N2], seed=0)
    Xa, W1a, W2b = X.to(pl.a), W1.to(pl.a), W2.to(pl.b)
    # the same kernels run without the protocol, one after the other
    Y1s = torch.empty(M, N1, dtype=torch.bfloat16, device=pl.a)
    pl.ext.gemm_tma(Xa, W1a, Y1s, cfg1)
    Y1s_b = Y1s.to(pl.b)
    Y2s = torch.empty(M, N2, dtype=torch.bfloat16, device=pl.b)
    with torch.cuda.device(pl.b):
        pl.ext.gemm_tma(Y1s_b, W2b, Y2s, cfg2)
    torch.cuda.synchronize(pl.a); torch.cuda.synchronize(pl.b)
    for r in range(runs):
        with torch.cuda.device(pl.b):
            pl.Y1.fill_(float("nan")); pl.Y2.fill_(float("nan"))
        torch.cuda.synchronize(pl.b)
        pl.run(Xa, W1a, W2b)
        pl.check()
        assert torch.equal(pl.Y1, Y1s_b), f"run {r}: pipelined Y1 differs from the sequential run in {(pl.Y1 != Y1s_b).sum().item()} elements"
        assert torch.equal(pl.Y2, Y2s), f"run {r}: pipelined Y2 differs from the sequential run in {(pl.Y2 != Y2s).sum().item()} elements"
        BM2, BN2 = pl.tile(cfg2)
        C = -(-M // BM2) * pl.tn2
        bad = oc.check_link_invariants(pl.src_b.cpu().numpy(), int(pl.tail_b.item()), pl.sb.cpu().numpy(), C, pl.tn2, bool(pl.rowpanel))
        assert bad == [], bad
        assert int(pl.head_a.item()) >= pl.src_a.numel() and int(pl.head_b.item()) >= C
    return pl, X, W1, W2


@pytest.mark.parametrize("case", [(256, 512, 512, 768, 3, 3, {}), (512, 1024, 1024, 1024, 5, 3, dict(group_rows=2)),
                                  (512, 512, 1024, 768, 10, 10, {}), (768, 512, 768, 1024, 10, 3, dict(group_rows=2)), (640, 256, 512, 512, 3, 10, dict(scoreboard="tile")),
                                  (384, 512, 512, 512, 10, 10, dict(group_rows=1)),
                                  (768, 512, 1024, 1536, 11, 11, dict(group_rows=2)), (512, 256, 1280, 768, 10, 11, {}), (1024, 512, 1024, 512, 11, 3, dict(group_rows="head")),
                                  (2048, 512, 512, 768, 3, 3, dict(group_rows="ramp")), (2304, 256, 768, 512, 10, 10, dict(group_rows=[1, 3, 4, 1])),
                                  (384, 512, 768, 512, 3, 5, dict(scoreboard="tile")), (1000, 520, 1000, 264, 5, 5, dict(group_rows=8))])
def test_chain_one_gpu_small(case):
    M, K, N1, N2, c1, c2, kw = case
    pl, X, W1, W2 = _run_case(M, K, N1, N2, c1, c2, 0, 0, **kw)
    ref = oc.chain_reference(X, [W1, W2])
    mx, mean = oc.error_stats(pl.Y2.cpu(), ref)
    assert mx <= 2e-2 and mean <= 1e-3, (mx, mean)


@pytest.mark.parametrize("cfg,group_rows", [(3, 8), (10, 4), (11, 4), (11, 8), (11, "head")])
def test_chain_one_gpu_headline_config_vs_oracle(cfg, group_rows):
    """M=1024, N=K=8192 (the CPU-checkable configuration) on 128x256 tiles, CTA-pair 256x256 tiles and the benchmark's CTA-pair
    256x512 tiles, in the producer orders the benchmark uses (groups of 8 tile rows; head-ramped groups)."""
    pl, X, W1, W2 = _run_case(1024, 8192, 8192, 8192, cfg, cfg, 0, 0, runs=2, fence=1, group_rows=group_rows)
    ys = oc.chain_reference(X, [W1, W2], keep=True)
    for got, ref, name in ((pl.Y1, ys[0], "Y1"), (pl.Y2, ys[1], "Y2")):
        mx, mean = oc.error_stats(got.cpu(), ref)
        assert mx <= 2e-2 and mean <= 1e-3, (name, mx, mean)


@pytest.mark.parametrize("cfg", [3, 10])
@pytest.mark.parametrize("rowpanel", [True, False])
def test_chain_serialised_order_is_bit_exact(rowpanel, cfg):
    """With a one-CTA producer the order in which consumer work becomes ready is deterministic: the queue must equal
    the sequential protocol model's, entry for entry."""
    from ctapp.pipeline import Chain
    M, K, N1, N2 = 512, 256, 1024, 768
    BMt = 256 if cfg == 10 else 128
    ch = Chain(M, K, [N1, N2], [0, 0], cfg=cfg, group_rows=2, scoreboard="rowpanel" if rowpanel else "tile", sms=2 if cfg == 10 else 1)
    X, Ws = oc.make_chain_inputs(M, K, [N1, N2], seed=1)
    ch.run(X.cuda(), [w.cuda() for w in Ws])
    ch.check()
    entries, tail, sb = oc.simulate_link(M, N1, N2, BMt, 256, BMt, 256, rowpanel, 2)
    assert np.array_equal(ch.entries[1].cpu().numpy(), entries)
    assert int(ch.tail[1].item()) == tail
    assert np.array_equal(ch.sb[0].cpu().numpy(), sb)
    mx, mean = oc.error_stats(ch.Y[1].cpu(), oc.chain_reference(X, Ws))
    assert mx <= 2e-2 and mean <= 1e-3


def _kchunk_case(M, K, N1, N2, cfg1, cfg2, devA, devB, group_rows, runs=3):
    """A two-stage chain with k-chunk dependencies: both outputs bit-identical to the same kernels run one after the other, every
    flag == the run's number afterwards (the oracle's model of the link), every tile taken exactly once."""
    from ctapp.pipeline import Pipeline
    pl = Pipeline(M, K, N1, N2, cfg1, cfg2, devA=devA, devB=devB, group_rows=group_rows, scoreboard="kchunk")
    ch = pl.chain
    X, (W1, W2) = oc.make_chain_inputs(M, K, [N1, N2], seed=0)
    Xa, W1a, W2b = X.to(pl.a), W1.to(pl.a), W2.to(pl.b)
    Y1s = torch.empty(M, N1, dtype=torch.bfloat16, device=pl.a)
    pl.ext.gemm_tma(Xa, W1a, Y1s, cfg1)
    Y1s_b = Y1s.to(pl.b)
    Y2s = torch.empty(M, N2, dtype=torch.bfloat16, device=pl.b)
    with torch.cuda.device(pl.b):
        pl.ext.gemm_tma(Y1s_b, W2b, Y2s, cfg2)
    torch.cuda.synchronize(pl.a); torch.cuda.synchronize(pl.b)
    BM, BN1 = pl.tile(cfg1)
    for r in range(1, runs + 1):
        with torch.cuda.device(pl.b):
            pl.Y1.fill_(float("nan")); pl.Y2.fill_(float("nan"))
        torch.cuda.synchronize(pl.b)
        pl.run(Xa, W1a, W2b)
        pl.check()
        assert torch.equal(pl.Y1, Y1s_b) and torch.equal(pl.Y2, Y2s), f"run {r}: the streamed chain differs from the sequential one"
        flags, need = oc.simulate_kchunk_link(ch.entries[0].cpu().numpy(), ch.tn[0], ch.entries[1].cpu().numpy(), ch.tn[1], -(-N1 // BN1), run_id=r)
        assert np.array_equal(ch.chunk[1].cpu().numpy(), flags)
        assert need.max() <= ch.ntiles[0]
        assert int(ch.head[0].item()) >= ch.ntiles[0] and int(ch.head[1].item()) >= ch.ntiles[1]
    return pl, X, W1, W2


@pytest.mark.parametrize("case", [(512, 512, 1024, 768, 10, 10, 2), (768, 256, 1536, 1024, 10, 11, 2), (1024, 512, 1024, 1024, 11, 11, 4),
                                  (640, 512, 768, 512, 3, 3, 2), (1024, 256, 1024, 512, 11, 10, "head"), (384, 512, 520, 264, 5, 5, 0)])
def test_chain_kchunk_one_gpu(case):
    M, K, N1, N2, c1, c2, g = case
    pl, X, W1, W2 = _kchunk_case(M, K, N1, N2, c1, c2, 0, 0, g)
    mx, mean = oc.error_stats(pl.Y2.cpu(), oc.chain_reference(X, [W1, W2]))
    assert mx <= 2e-2 and mean <= 1e-3, (mx, mean)


def test_chain_kchunk_three_stages_one_gpu():
    from ctapp.pipeline import Chain
    M, K, widths = 512, 512, [768, 1024, 512]
    ch = Chain(M, K, widths, [0, 0, 0], cfg=[10, 11, 10], group_rows=2, scoreboard="kchunk")
    X, Ws = oc.make_chain_inputs(M, K, widths, seed=4)
    for _ in range(2):
        ch.run(X.cuda(), [w.cuda() for w in Ws])
        ch.check()
    mx, mean = oc.error_stats(ch.Y[-1].cpu(), oc.chain_reference(X, Ws))
    assert mx <= 2e-2 and mean <= 1e-3, (mx, mean)
    assert all(int(c.min().item()) == 2 for c in ch.chunk[1:])


def test_kchunk_consumer_without_producer_times_out_cleanly():
    """Host-side fault injection: a consuming stage whose k-chunk flags nobody raises gives up (code 8) and the context lives on."""
    from ctapp.ext import load, new_status
    ext = load()
    ext.set_wait_limit_ms(50)
    try:
        M, K, N = 256, 256, 512
        X = torch.zeros(M, K, dtype=torch.bfloat16, device="cuda"); W = torch.zeros(N, K, dtype=torch.bfloat16, device="cuda")
        Y = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        entries = torch.arange(2, dtype=torch.int32, device="cuda")
        head = torch.zeros(1, dtype=torch.int32, device="cuda"); tail = torch.full((1,), 2, dtype=torch.int32, device="cuda")
        flags = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
        status = new_status("cuda")
        ext.ctapp_gemm(X, W, Y, 10, entries, head, tail, None, None, None, None, None, None, 2, 0, 0, status=status, chunk_src=flags, chunk_kblocks=4,
                       chunk_value=1)
        torch.cuda.synchronize()
        s = status.cpu().tolist()
        assert s[0] == 8 and s[3] == 1, s
        ext.gemm_tma(X, W, Y, 10)
        torch.cuda.synchronize()
    finally:
        ext.set_wait_limit_ms(2000)


def test_chain_three_stages_one_gpu():
    from ctapp.pipeline import Chain
    M, K, widths = 384, 512, [768, 512, 1024]
    ch = Chain(M, K, widths, [0, 0, 0], cfg=[3, 5, 3], group_rows=4)
    X, Ws = oc.make_chain_inputs(M, K, widths, seed=2)
    for _ in range(2):
        ch.run(X.cuda(), [w.cuda() for w in Ws])
        ch.check()
    mx, mean = oc.error_stats(ch.Y[-1].cpu(), oc.chain_reference(X, Ws))
    assert mx <= 2e-2 and mean <= 1e-3, (mx, mean)


def test_gantt_of_a_one_gpu_chain_run():
    """Stamps of a two-stage run on one GPU drawn as SVG: every CTA of both stages gets a row."""
    import xml.dom.minidom
    from ctapp.pipeline import Chain
    from ctapp.timeline import chain_gantt_svg
    M, K, N = 1024, 1024, 2048
    ch = Chain(M, K, [N, N], [0, 0], cfg=10, group_rows=2, stamps=True)
    X, Ws = oc.make_chain_inputs(M, K, [N, N], seed=0)
    ch.run(X.cuda(0), [w.cuda(0) for w in Ws])
    ch.check()
    svg = chain_gantt_svg(ch)
    xml.dom.minidom.parseString(svg)
    ctas = 2 * min(148 // 2, (M // 256) * (N // 256)) * 2          # CTA pairs that got a tile, both stages
    assert f"{ctas} CTAs" in svg, svg[:200]


def test_missing_producer_times_out_cleanly():
    """Fault injection on the host side: the consumer is launched although nothing will ever fill its queue.  Its bounded
    wait must give up, report code 1 in the status buffer, and leave the context usable."""
    from ctapp.ext import load, new_status
    ext = load()
    ext.set_wait_limit_ms(50)
    try:
        M, K, N = 256, 256, 512
        X = torch.zeros(M, K, dtype=torch.bfloat16, device="cuda"); W = torch.zeros(N, K, dtype=torch.bfloat16, device="cuda")
        Y = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        ntiles = 2 * 2
        entries = torch.full((ntiles,), -1, dtype=torch.int32, device="cuda")
        head = torch.zeros(1, dtype=torch.int32, device="cuda"); tail = torch.zeros(1, dtype=torch.int32, device="cuda")
        status = new_status("cuda")
        ext.ctapp_gemm(X, W, Y, 3, entries, head, tail, None, None, None, None, None, None, 2, 0, 0, status=status)
        torch.cuda.synchronize()
        s = status.cpu().tolist()
        assert s[0] == 1 and s[5] >= 1, s
        # the context still works
        Y2 = torch.empty_like(Y)
        ext.gemm_tma(X, W, Y2, 3)
        torch.cuda.synchronize()
        assert torch.equal(Y2, torch.zeros_like(Y2))
    finally:
        ext.set_wait_limit_ms(2000)


@pytest.mark.multigpu(2)
@pytest.mark.parametrize("case", [(1024, 8192, 8192, 8192, 3, 3, dict(fence=1, group_rows=8)), (4096, 8192, 8192, 8192, 3, 3, dict(fence=1, group_rows=8)),
                                  (1024, 8192, 8192, 8192, 10, 10, dict(fence=1, group_rows=4)), (4096, 8192, 8192, 8192, 10, 10, dict(fence=1, group_rows=8)),
                                  (4096, 8192, 8192, 8192, 10, 3, dict(fence=1, group_rows=8)),
                                  (4096, 4096, 8192, 4096, 5, 3, dict(fence=1)), (2048, 8192, 8192, 10240, 3, 3, dict(scoreboard="tile", group_rows=8))])
def test_chain_two_gpus(case):
    M, K, N1, N2, c1, c2, kw = case
    pl, X, W1, W2 = _run_case(M, K, N1, N2, c1, c2, 0, 1, runs=10, **kw)
    if M <= 1024:
        mx, mean = oc.error_stats(pl.Y2.cpu(), oc.chain_reference(X, [W1, W2]))
        assert mx <= 2e-2 and mean <= 1e-3, (mx, mean)


@pytest.mark.multigpu(2)
@pytest.mark.parametrize("case", [(4096, 8192, 8192, 8192, 10, 10, 4), (4096, 8192, 8192, 8192, 10, 11, 4), (8192, 8192, 8192, 8192, 11, 11, 8),
                                  (1024, 8192, 8192, 8192, 10, 10, 2)])
def test_chain_kchunk_two_gpus(case):
    """Producer and consumer really overlap: the consumer's main loops stream behind the producer's tiles."""
    M, K, N1, N2, c1, c2, g = case
    pl, X, W1, W2 = _kchunk_case(M, K, N1, N2, c1, c2, 0, 1, g, runs=8)
    if M <= 1024:
        mx, mean = oc.error_stats(pl.Y2.cpu(), oc.chain_reference(X, [W1, W2]))
        assert mx <= 2e-2 and mean <= 1e-3, (mx, mean)


@pytest.mark.multigpu(2)
def test_kchunk_negative_control_two_gpus():
    """skip_wait makes the consumer ignore the k-chunk flags: it must then read rows that have not arrived."""
    from ctapp.pipeline import Pipeline
    M, K, N = 8192, 8192, 8192
    pl = Pipeline(M, K, N, N, 10, 10, devA=0, devB=1, skip_wait=1, group_rows=4, scoreboard="kchunk")
    X, (W1, W2) = oc.make_chain_inputs(M, K, [N, N], seed=0)
    with torch.cuda.device(pl.b):
        pl.Y1.fill_(float("nan"))
    torch.cuda.synchronize(pl.b)
    pl.run(X.to(pl.a), W1.to(pl.a), W2.to(pl.b))
    pl.check()
    assert torch.isnan(pl.Y2.float()).any(), "skipping the waits changed nothing: the test cannot see races"


@pytest.mark.multigpu(2)
def test_negative_control_two_gpus():
    """skip_wait makes the consumer ignore the queue; its output must then differ from the correct one somewhere, which shows
    the comparison above can see a race."""
    from ctapp.pipeline import Pipeline
    M, K, N = 8192, 8192, 8192
    pl = Pipeline(M, K, N, N, 3, 3, devA=0, devB=1, skip_wait=1, fence=1, group_rows=8)
    g = torch.Generator().manual_seed(0)
    X = torch.randn(M, K, generator=g).to(torch.bfloat16).to(pl.a)
    W1 = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(pl.a)
    W2 = (torch.randn(N, N, generator=g) / N ** 0.5).to(torch.bfloat16).to(pl.b)
    with torch.cuda.device(pl.b):
        pl.Y1.fill_(float("nan"))
    torch.cuda.synchronize(pl.b)
    pl.run(X, W1, W2)
    pl.check()
    assert torch.isnan(pl.Y2.float()).any(), "skipping the wait changed nothing: the test cannot see races"


@pytest.mark.multigpu(2)
def test_gated_harness_and_methods_two_gpus():
    """The comparison methods give the chain's result (micro-batching bit for bit: same library GEMM on row slices; tensor
    parallelism within bf16 tolerance), and the gate really holds the GPUs: a slow host between gate and launch does not
    change the measured time."""
    import time
    from ctapp import methods as mt
    from ctapp.timing import measure
    M, N = 1024, 2048
    g = torch.Generator().manual_seed(0)
    X = torch.randn(M, N, generator=g).to(torch.bfloat16).to(mt.dev(0))
    W1 = (torch.randn(N, N, generator=g) / N ** 0.5).to(torch.bfloat16)
    W2 = (torch.randn(N, N, generator=g) / N ** 0.5).to(torch.bfloat16)
    one = mt.OneGpuCublas(M, X, W1.to(mt.dev(0)), W2.to(mt.dev(0)))
    one.enqueue(); torch.cuda.synchronize(0)
    ref = one.result().cpu()
    mb = mt.MicroBatchCublas(M, X, W1.to(mt.dev(0)), W2.to(mt.dev(1)), 256)
    mb.enqueue(); torch.cuda.synchronize(0); torch.cuda.synchronize(1)
    mx, mean = oc.error_stats(mb.result().cpu(), ref)
    assert mx <= 2e-2 and mean <= 1e-3
    tp = mt.TensorParallel2(M, X, W1.to(mt.dev(0)), W2.to(mt.dev(1)))
    tp.enqueue(); torch.cuda.synchronize(0); torch.cuda.synchronize(1)
    mx, mean = oc.error_stats(tp.result().cpu(), ref)
    assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)
    ct = mt.Ctapp(M, X, W1.to(mt.dev(0)), W2.to(mt.dev(1)), 10, 10, 2)
    t_fast = measure(ct, reps=5, warmup=2)[0]
    ct.pl.check()
    mx, mean = oc.error_stats(ct.result().cpu(), ref)
    assert mx <= 2e-2 and mean <= 1e-3, (mx, mean)

    class SlowHost(mt.Ctapp):
        def enqueue(self):
            time.sleep(0.01)
            super().enqueue()
    slow = SlowHost(M, X, W1.to(mt.dev(0)), W2.to(mt.dev(1)), 10, 10, 2)
    t_slow = measure(slow, reps=5, warmup=2)[0]
    assert t_slow < 3 * t_fast + 200, (t_fast, t_slow)     # microseconds: the 10 ms host sleep is outside the window


@pytest.mark.multigpu(2)
def test_clock_offset_and_chain_timeline_two_gpus():
    """The bounded flag ping-pong between two GPUs gives a stable clock offset and a round trip of a few microseconds, and the
    per-CTA stamps of a pipelined run, put on one clock, tell the pipelining story: the consumer is resident from the start, gets
    its first tile only after the producer has published, and finishes after the producer."""
    from ctapp.pipeline import Chain
    from ctapp.timeline import chain_timeline, clock_offset
    off1, rtt1 = clock_offset(0, 1)
    off2, rtt2 = clock_offset(0, 1)
    assert 500 < rtt1 < 50000 and 500 < rtt2 < 50000, (rtt1, rtt2)       # ns
    assert abs(off1 - off2) < 5000, (off1, off2)
    M, K, N = 4096, 8192, 8192
    ch = Chain(M, K, [N, N], [0, 1], cfg=10, group_rows=2, stamps=True)
    X, Ws = oc.make_chain_inputs(M, K, [N, N], seed=0)
    Xa, Wd = X.cuda(0), [Ws[0].cuda(0), Ws[1].cuda(1)]
    for _ in range(2):
        ch.run(Xa, Wd)
        ch.check()
    tl = chain_timeline(ch)
    p, c = tl
    # 16 pair-rows x 32 n-tiles; both CTAs of a pair count the pair's tiles
    assert p["ctas"] == 148 and c["ctas"] == 148 and p["tiles"] == 2 * 16 * 32 and c["tiles"] == 2 * 16 * 32
    assert c["first_tile_min_us"] > p["first_tile_min_us"] + 5, (p, c)     # nothing to consume before the first panel is published
    assert c["exit_max_us"] > p["exit_max_us"], (p, c)
    assert c["first_tile_min_us"] < p["exit_max_us"], "the consumer started only after the producer had finished: no pipelining"
    from ctapp.timeline import chain_gantt_svg
    svg = chain_gantt_svg(ch)
    assert svg.count("<rect") >= 2 * 148 * 3 and "stage 1 gpu 1" in svg


@pytest.mark.multigpu(2)
@pytest.mark.parametrize("cfg", [3, 10])
def test_chain_stages_one_process_per_gpu_overlapped_steps(cfg):
    """One stage per process (the form ``bench.py --gpus N`` runs): five steps with different inputs enqueued back to back;
    the doubled links let step e+1 enter a link while step e is still being consumed, and every step's result must be
    the oracle's."""
    import mp_cases
    from ctapp.tp4 import launch
    world = 4 if torch.cuda.device_count() >= 4 else 2
    res, bad = launch(mp_cases.chain_stages_case, world, 29741 + cfg, 1024, 2048, 5, cfg, 2 if cfg == 3 else "head")
    assert not bad, res
    assert all(r == [] for r in res), res


@pytest.mark.multigpu(2)
@pytest.mark.parametrize("cfg,group_rows", [(11, 4), (10, 2), (3, 4)])
def test_chain_stages_kchunk_one_process_per_gpu(cfg, group_rows):
    """The same with k-chunk flags on every link: no queue, no scoreboard, flags that carry the step number (six steps, so
    that either set of every doubled link is used three times)."""
    import mp_cases
    from ctapp.tp4 import launch
    world = 4 if torch.cuda.device_count() >= 4 else 2
    res, bad = launch(mp_cases.chain_stages_case, world, 29761 + cfg, 1024, 2048, 6, cfg, group_rows, "kchunk")
    assert not bad, res
    assert all(r == [] for r in res), res
