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
    o = producer_order(32 * 32, 32, "ramp")
    assert sorted(o.tolist()) == list(range(1024))
    assert o[:32].tolist() == list(range(32))                      # first group: one tile row, n ascending
    assert torch.equal(producer_order(64, 4, [4, 4, 4, 4]), producer_order(64, 4, 4))
    o = producer_order(16 * 4, 4, [1, 3, 4, 8])
    assert o[:4].tolist() == [0, 1, 2, 3] and o[4:7].tolist() == [4, 8, 12]      # second group: rows 1-3, n-major


def test_boundary_tail_rule_matches_oracle():
    """``CtappBoundary._tail`` (host logic, no GPU needed for the rule itself) against the oracle's statement of it."""
    from oracle import boundary as ob
    import types
    from ctapp.tp4 import CtappBoundary
    for M in (128, 1920, 2048, 4096, 16384):
        for raster, swz, down_tail in ((1, 1, "auto"), (2, 1, "auto"), (1, 2, "auto"), (1, 1, 5), (1, 1, 32)):
            fake = types.SimpleNamespace(down_tail=down_tail, down_raster=raster, down_swizzle=swz, n1=8192)
            want = down_tail if down_tail != "auto" else ob.tail_cols(M, raster, swz)
            assert CtappBoundary._tail(fake, M) == want
