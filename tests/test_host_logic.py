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
