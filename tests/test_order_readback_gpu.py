"""The integer maps the kernels schedule by, read back from the device and compared entry for entry with the oracle's
restatement of the reference's functions (``tp4_remap_tile``, csrc/ctapp_tp4.cuh:897-906; ``red5_map``, :551-565; the grouped
producer order, ctapp/pipeline.py:48-51).  Two kinds of read-back:

  * the device functions themselves (``decode_tile``, ``unit_map``, ``queue_slot``) evaluated for every index by a small kernel;
  * the order a real launch works in: a producer GEMM on one CTA (pair) and an owner reducer of one warp append every tile /
    unit they take to a log, which must be the oracle's sequence.  With more CTAs the global order depends on timing, so the
    exact comparison is made in this serialised form.
"""
import numpy as np
import pytest
import torch

from oracle import boundary as ob
from oracle import chain as oc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("TM,TN,tail", [(32, 32, 16), (8, 32, 8), (5, 7, 3), (16, 32, 0), (1, 4, 4), (33, 20, 20)])
def test_tail_remap_matches_the_oracle(TM, TN, tail):
    from ctapp.ext import load
    got = load().debug_tile_order(1, TM, TN, tail_cols=tail).numpy()
    want = np.array([ob.remap_tile(L, TM, TN, tail) for L in range(TM * TN)], dtype=np.int32)
    assert np.array_equal(got, want)
    assert sorted(map(tuple, got.tolist())) == [(m, n) for m in range(TM) for n in range(TN)]          # a bijection onto the tile grid


@pytest.mark.parametrize("TM,TN,g", [(32, 32, 8), (16, 16, 4), (7, 5, 3), (9, 4, 1), (3, 8, 16)])
def test_grouped_and_row_major_orders_match_the_oracle(TM, TN, g):
    from ctapp.ext import load
    ext = load()
    got = ext.debug_tile_order(0, TM, TN, group_rows=g).numpy()
    assert np.array_equal(got, np.array(ob.tile_order(0, TM, TN, g), dtype=np.int32))
    # the same order as a list of tile ids is what the chain's first stage is given (reference ctapp/pipeline.py:48-51)
    assert np.array_equal(got[:, 0] * TN + got[:, 1], oc.producer_order(TM * TN, TN, g))
    got2 = ext.debug_tile_order(2, TM, TN).numpy()
    assert np.array_equal(got2, np.array(ob.tile_order(2, TM, TN), dtype=np.int32))


@pytest.mark.parametrize("Pr,tn,tail,order,swz", [(8, 32, 16, 1, 1), (2, 32, 8, 1, 1), (4, 32, 0, 1, 1), (4, 32, 0, 1, 2), (3, 8, 0, 1, 4),
                                                 (8, 32, 0, 2, 1), (1, 2, 2, 1, 1), (5, 6, 0, 2, 1)])
def test_unit_map_matches_the_oracle(Pr, tn, tail, order, swz):
    from ctapp.ext import load
    got = load().debug_unit_order(Pr, tn, tail, order, swz).numpy()
    want = np.array([ob.unit_map(u, Pr, tn, tail, order, swz) for u in range(Pr * tn * 4)], dtype=np.int32)
    assert np.array_equal(got, want)
    assert len({tuple(r) for r in got.tolist()}) == Pr * tn * 4


@pytest.mark.parametrize("tm,tn,group", [(32, 16, 8), (32, 32, 0), (10, 4, 3), (32, 16, [2, 4, 8, 8, 8, 2]), (7, 3, [1, 1, 2, 3])])
def test_queue_slots_match_the_host_model(tm, tn, group):
    from ctapp.ext import load
    from ctapp.pipeline import _window_args, pop_slots
    g, win = _window_args(group, torch.device("cuda", 0))
    got = load().debug_queue_slots(tm * tn, tn, src_group=g, src_windows=win).numpy()
    want = pop_slots(tm * tn, tn, group).numpy()
    assert np.array_equal(got, want)
    assert sorted(got.tolist()) == list(range(tm * tn))


@pytest.mark.parametrize("cta_pair", [True, False])
@pytest.mark.parametrize("M,tail", [(1024, "auto"), (2048, "auto"), (768, 0), (512, 2)])
def test_one_cta_producer_walks_the_oracle_order(M, tail, cta_pair):
    """Producer GEMM (mode 7) on a single CTA (or CTA pair): the tiles it takes, in order, and the unit order of a one-warp
    owner reducer behind it, against the oracle; then the step's results against the oracle's model as usual."""
    from ctapp.symm import LocalGroup
    from ctapp.tp4 import CtappBoundary
    K, n1, N2_ = 256, 1024, 256
    tn = n1 // 256
    bd = CtappBoundary(M, K, N2_, 0, 1, LocalGroup([0]), torch.device("cuda", 0), protocol="v5", n1=n1, fusion="serial", cta_pair=cta_pair,
                       down_tail=tail, red_blocks=1, red_threads=32)
    Wd, gamma, Wq = ob.make_weights(seed=2, K=K, N2_=N2_, n1=n1)
    h, resid = ob.make_inputs(M, seed=3, K=K, n1=n1)
    wd, _, wqf = ob.shard_weights(Wd, Wq, gamma, 0, 1)
    TM = M // 256 if cta_pair else M // 128          # tile rows of the schedule
    tile_log = torch.zeros(1 + TM * tn, dtype=torch.int32, device="cuda")
    unit_log = torch.zeros(1 + (M // 128) * tn * 4, dtype=torch.int32, device="cuda")
    bd.epoch += 1
    bd._last = (bd.epoch & 1, M)
    bd._step(M)
    bd.launch_producer(h.cuda(), wd.cuda(), M, tile_log=tile_log, sms=2 if cta_pair else 1)
    bd.launch_reducer(M, resid.cuda(), bd.epoch & 1, unit_log=unit_log)
    bd.launch_consumer(wqf.cuda(), M, bd.epoch & 1)
    bd.check()
    C = bd.tail_cols(M)
    tl = tile_log.cpu().numpy()
    assert tl[0] == TM * tn
    got = np.stack([tl[1:] >> 16, tl[1:] & 0xffff], axis=1)
    want = np.array([ob.remap_tile(L, TM, tn, C) for L in range(TM * tn)], dtype=np.int32)
    assert np.array_equal(got, want), (got[:8], want[:8])
    ul = unit_log.cpu().numpy()
    U = (M // 128) * tn * 4
    assert ul[0] == U
    gotu = np.stack([ul[1:] >> 16, (ul[1:] >> 2) & 0x3fff, ul[1:] & 3], axis=1)
    wantu = np.array([ob.unit_map(u, M // 128, tn, C) for u in range(U)], dtype=np.int32)
    assert np.array_equal(gotu, wantu), (gotu[:8], wantu[:8])
    x_model, out_model = ob.boundary_device_model(h, Wd, resid, gamma, Wq, 1)
    ulp = lambda a, b: ((a.view(torch.int16).int() - b.view(torch.int16).int()).abs() <= 1).float().mean().item()  # noqa: E731
    assert ulp(bd.x().cpu(), x_model) >= 0.99 and ulp(bd._out_full[:M].cpu(), out_model) >= 0.98
