"""Host-side logic of the product package against the oracle (no GPU)."""
import numpy as np
import pytest

from oracle import chain as oc


@pytest.mark.parametrize("case", [(1024, 8192, 8192, 128, 128, 128, 128, True), (1024, 8192, 8192, 128, 256, 128, 256, True),
                                  (4096, 8192, 8192, 128, 128, 64, 256, True), (4096, 8192, 10240, 128, 128, 64, 256, False),
                                  (1000, 1000, 520, 64, 256, 128, 128, False), (130, 300, 300, 128, 128, 128, 128, False),
                                  (128, 256, 256, 128, 256, 128, 256, True)])
def test_build_deps_equals_oracle(case):
    from ctapp.pipeline import build_deps
    got = build_deps(*case)
    ref = oc.build_deps(*case[:7], rowpanel=case[7])
    for g, r in zip(got, ref):
        assert g.dtype.is_floating_point is False and np.array_equal(g.numpy(), r)


@pytest.mark.parametrize("P,tn,g", [(512, 64, 8), (256, 32, 8), (96, 32, 2), (160, 32, 4), (64, 64, 0)])
def test_producer_order_equals_oracle(P, tn, g):
    from ctapp.pipeline import producer_order
    assert np.array_equal(producer_order(P, tn, g).numpy(), oc.producer_order(P, tn, g))


def test_ramped_and_listed_producer_orders():
    import torch
    from ctapp.pipeline import producer_order, ramp_groups
    for tm in (1, 2, 3, 5, 8, 16, 32, 33, 64, 128):
        g = ramp_groups(tm)
        assert sum(g) == tm and all(1 <= v <= 8 for v in g) and g[0] == 1 and g[-1] == 1
    from ctapp.pipeline import head_groups
    assert head_groups(32) == [2, 4, 8, 8, 8, 2] and head_groups(1) == [1] and head_groups(3) == [2, 1] and head_groups(11) == [2, 4, 5]
    assert sorted(producer_order(11 * 4, 4, "head").tolist()) == list(range(44))
    o = producer_order(32 * 32, 32, "ramp")
    assert sorted(o.tolist()) == list(range(1024))
    assert o[:32].tolist() == list(range(32))                      # first group: one tile row, n ascending
    assert torch.equal(producer_order(64, 4, [4, 4, 4, 4]), producer_order(64, 4, 4))
    o = producer_order(16 * 4, 4, [1, 3, 4, 8])
    assert o[:4].tolist() == [0, 1, 2, 3] and o[4:7].tolist() == [4, 8, 12]      # second group: rows 1-3, n-major


@pytest.mark.parametrize("tm,tn,g", [(32, 32, 8), (16, 32, 2), (5, 4, 2), (7, 3, 4), (3, 8, 8), (4, 4, 1), (4, 4, 0)])
def test_consumer_pop_windows_are_a_permutation_in_n_major_order(tm, tn, g):
    """The i-th pop of a consuming stage reads slot pop_slots[i]: every slot exactly once; inside a window of g published
    row panels the pops take slot j of every panel before slot j+1; when the producer publishes its groups in order, the
    resulting tile order is the producer's own grouped order."""
    from ctapp.pipeline import consumer_window, pop_slots, producer_order
    n = tm * tn
    slots = pop_slots(n, tn, g).numpy()
    assert sorted(slots.tolist()) == list(range(n))
    if g <= 1:
        assert slots.tolist() == list(range(n))
        return
    panel, j = slots // tn, slots % tn
    for w0 in range(0, tm, g):
        gw = min(g, tm - w0)
        sel = (panel >= w0) & (panel < w0 + gw)
        idx = np.nonzero(sel)[0]
        assert idx.min() == w0 * tn and idx.max() == (w0 + gw) * tn - 1          # a window's pops are consecutive
        assert np.array_equal(j[idx], np.repeat(np.arange(tn), gw))              # n-tile major ...
        assert np.array_equal(panel[idx], np.tile(np.arange(w0, w0 + gw), tn))   # ... over the window's panels
    # queue filled panel by panel in ascending order (entry = panel * tn + j): tiles come out in the grouped producer order
    if tm % g == 0:
        assert np.array_equal(slots, producer_order(n, tn, g).numpy())
    # windows of varying size follow a ramped producer the same way
    from ctapp.pipeline import ramp_groups
    sizes = ramp_groups(tm)
    assert np.array_equal(pop_slots(n, tn, sizes).numpy(), producer_order(n, tn, sizes).numpy())
    assert consumer_window("ramp", 1, 256, 256, tm) == sizes and consumer_window([1, tm - 1], 1, 128, 128, tm) == [1, tm - 1]
    assert consumer_window("ramp", 1, 128, 256, tm) == 0
    assert consumer_window(8, 1, 256, 256) == 8 and consumer_window(8, 1, 128, 256) == 4 and consumer_window(2, 1, 128, 256) == 0
    assert consumer_window(8, 0, 256, 256) == 0 and consumer_window(0, 1, 128, 128) == 0


def test_boundary_tail_rule_matches_oracle():
    """``CtappBoundary.tail_cols`` (host logic, no GPU needed for the rule itself) against the oracle's statement of it."""
    from oracle import boundary as ob
    import types
    from ctapp.tp4 import CtappBoundary
    for M in (128, 1920, 2048, 4096, 16384):
        for raster, swz, down_tail in ((1, 1, "auto"), (2, 1, "auto"), (1, 2, "auto"), (1, 1, 5), (1, 1, 32)):
            fake = types.SimpleNamespace(down_tail=down_tail, down_raster=raster, down_swizzle=swz, n1=8192)
            want = down_tail if down_tail != "auto" else ob.tail_cols(M, raster, swz)
            assert CtappBoundary.tail_cols(fake, M) == want


def test_gantt_svg_from_synthetic_stamps(tmp_path):
    """The Gantt writer needs no GPU: rows = CTAs that ran, ordered by SM id, second stage shifted by its clock offset."""
    import torch
    import xml.dom.minidom
    from ctapp.timeline import gantt_svg
    a = torch.zeros(4, 8, dtype=torch.int64)
    a[0] = torch.tensor([1000, 1100, 5000, 5200, 5300, 7, 3, 5400])
    a[1] = torch.tensor([1005, 1110, 5100, 5300, 5400, 7, 1, 5500])
    a[2] = torch.tensor([1010, 0, 0, 0, 0, 0, 2, 1500])             # never got a tile
    b = torch.zeros(2, 8, dtype=torch.int64)
    b[0] = torch.tensor([90000, 91000, 95000, 95100, 0, 7, 0, 95200])  # other GPU's clock: 88 500 ns ahead
    text = gantt_svg([("stage 0", a, 0.0), ("stage 1", b, -88500.0)], str(tmp_path / "g.svg"))
    doc = xml.dom.minidom.parseString(text)
    assert doc.documentElement.tagName == "svg"
    assert "4 CTAs" in text and "stage 0" in text and "stage 1" in text
    assert text.count("<rect") == 3 * 4 + 1 + 4               # four segments for each of the 3 CTAs that worked, one idle row, legend
    assert (tmp_path / "g.svg").read_text() == text


def test_integer_artefacts_equal_the_oracle_on_random_shapes():
    """Seeded random shapes (ragged M, mixed tile sizes): CSR, scoreboard and producer order bit-exact against the oracle, the
    consumer pop windows a permutation that reproduces the producer's order, and the protocol model's invariants hold when
    the producer finishes tiles in that order."""
    import random
    import torch
    from ctapp.pipeline import build_deps, consumer_window, head_groups, pop_slots, producer_order, ramp_groups
    rnd = random.Random(1234)
    for _ in range(40):
        BM1, BM2 = rnd.choice([128, 256]), rnd.choice([128, 256])
        BN1, BN2 = rnd.choice([128, 256]), rnd.choice([128, 256])
        M = rnd.randrange(1, 24) * 64 + rnd.choice([0, 8, 40])
        N1, N2 = rnd.randrange(1, 9) * 128, rnd.randrange(1, 9) * 128
        rowpanel = rnd.random() < 0.7
        off, cons, sb = build_deps(M, N1, N2, BM1, BN1, BM2, BN2, rowpanel)
        o_off, o_cons, o_sb = oc.build_deps(M, N1, N2, BM1, BN1, BM2, BN2, rowpanel)
        assert np.array_equal(off.numpy(), o_off) and np.array_equal(cons.numpy(), o_cons) and np.array_equal(sb.numpy(), o_sb)
        tm1, tn1 = -(-M // BM1), -(-N1 // BN1)
        g = rnd.choice([0, 1, 2, 3, 4, 8])
        assert np.array_equal(producer_order(tm1 * tn1, tn1, g).numpy(), oc.producer_order(tm1 * tn1, tn1, g))
        for sizes in (head_groups(tm1), ramp_groups(tm1)):
            assert sum(sizes) == tm1 and all(s > 0 for s in sizes)
            order = producer_order(tm1 * tn1, tn1, sizes)
            assert sorted(order.tolist()) == list(range(tm1 * tn1))
            assert torch.equal(pop_slots(tm1 * tn1, tn1, sizes), order)
        entries, tail, sb_end = oc.simulate_link(M, N1, N2, BM1, BN1, BM2, BN2, rowpanel, group_rows=g)
        tm2, tn2 = -(-M // BM2), -(-N2 // BN2)
        assert oc.check_link_invariants(entries, tail, sb_end, tm2 * tn2, tn2, rowpanel) == []
        if rowpanel and g > 1:
            w = consumer_window(g, 1, BM1, BM2, tm2)
            slots = pop_slots(tm2 * tn2, tn2, w if w else 1).numpy()
            assert sorted(slots.tolist()) == list(range(tm2 * tn2))


def test_doubled_links_schedule_has_no_cycle_and_no_set_reuse():
    """Model of ``ChainStage``'s schedule for L ranks and E steps.  Kernels of a rank run in stream order: step e enqueues the
    reset that prepares the link set of step e+1 (and raises its ready flag upstream), then the GEMM of step e.  A GEMM cannot
    finish before its producer's GEMM of the same step has, and a producer cannot store step e before the consumer's reset for
    step e.  The dependency graph must be acyclic (nothing can wait for itself), and a link set (e & 1) must never be reset
    for step e+2 while the GEMM that reads step e from it can still be running."""
    from graphlib import TopologicalSorter
    L, E = 4, 7
    deps = {}

    def add(node, *before):
        deps.setdefault(node, set()).update(before)

    for g in range(L):
        prev = None
        stream = [("reset", g, 1)] + [op for e in range(1, E + 1) for op in (("reset", g, e + 1), ("gemm", g, e))]
        for op in stream:                                  # stream order on rank g
            add(op, *([prev] if prev else []))
            prev = op
        for e in range(1, E + 1):
            if g > 0:
                add(("gemm", g, e), ("gemm", g - 1, e))      # all of the producer's tiles of step e
                add(("gemm", g - 1, e), ("reset", g, e))     # the producer's first store of step e waits for this rank's ready flag
    order = list(TopologicalSorter(deps).static_order())    # raises CycleError on a deadlock
    pos = {op: i for i, op in enumerate(order)}
    for g in range(1, L):
        for e in range(1, E - 1):
            # the set of step e is prepared again for step e+2 only after this rank's GEMM of step e ...
            assert ("gemm", g, e) in deps[("reset", g, e + 2)] or pos[("gemm", g, e)] < pos[("reset", g, e + 2)]
            stream = [op for op in order if op[1] == g]
            assert stream.index(("gemm", g, e)) < stream.index(("reset", g, e + 2))
            # ... and the producer's step e+2, which writes that set, cannot start storing before that reset
            assert ("reset", g, e + 2) in deps[("gemm", g - 1, e + 2)]
    # at most two steps of a link are in flight: the producer's step e+2 needs the consumer's step e to be over
    assert all(pos[("gemm", g, e)] < pos[("gemm", g - 1, e + 2)] for g in range(1, L) for e in range(1, E - 1))


def test_producer_tile_choice_and_reducer_sm_defaults():
    """Host rules of ``CtappBoundary`` that need no GPU: the producer runs on 256 x 512 tiles only up to TP2 and only when every
    CTA pair still gets one; forced choices win; one CTA per tile stays one CTA per tile."""
    import types
    from ctapp.tp4 import CtappBoundary
    def pick(world, M, n1=8192, cta_pair=1, forced=None, sms=144):
        fake = types.SimpleNamespace(cta_pair=cta_pair, n1=n1, world=world, sms=sms, _down_wide=forced)
        return CtappBoundary.down_pair(fake, M)
    assert pick(2, 4096) == 2 and pick(1, 4096) == 2          # 16 x 16 tiles >= 72 pairs
    assert pick(2, 1024) == 1                                 # 4 x 16 tiles < 72 pairs
    assert pick(4, 4096) == 1 and pick(8, 8192) == 1          # coarser tiles reach the reducer later: narrow from TP4
    assert pick(4, 4096, forced=True) == 2 and pick(2, 4096, forced=False) == 1
    assert pick(2, 4096, n1=768) == 1                         # hidden size not a multiple of 512
    assert pick(2, 4096, cta_pair=0) == 0


def test_handover_model_orders_and_floor():
    """The timing model of a k-chunk link walks the same tile order as the host code, never ends before the producer plus one
    chunk, reproduces the figures quoted beside the measurements, and shows the lag behind a longer producer wave."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "cta-pipelining_b200", "bench"))
    import handover_model as hm
    from ctapp.pipeline import producer_order
    for tm, tn, g in [(16, 32, 4), (7, 5, 2), (3, 4, 8)]:
        want = producer_order(tm * tn, tn, g).tolist()
        assert [m * tn + n for m, n in hm.grouped_order(tm, tn, g)] == want
    for M in (1024, 4096, 8192):
        for g in (1, 2, 4, 8):
            tp, end = hm.link(M, group_rows=g)
            assert end >= tp + 97.0 / 32 - 1e-9
    assert [round(hm.link(M, group_rows=4)[1]) for M in (4096, 8192, 16384)] == [438, 814, 1505]
    # a producer on 256x512 tiles (100 us waves) that is 5 % faster per flop still hands over later than the 256x256 one
    tp_n, end_n = hm.link(8192, group_rows=4)
    tp_w, end_w = hm.link(8192, group_rows=4, tile_us=95.0, producer_bn=512)
    assert tp_w < tp_n and end_w > end_n
