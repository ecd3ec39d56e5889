"""One process per GPU (spawned): the NVLS multimem probes, and the boundary in its unicast and NVLS variants, against the
CPU oracle.  NCCL runs with NVLS off in these child processes; the library's own multimem stores are what is under test."""
import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu(2)]


def _world():
    import torch
    n = torch.cuda.device_count()
    return 8 if n >= 8 else 4 if n >= 4 else 2


def _run(fn, port, *args):
    from ctapp.tp4 import launch
    res, bad = launch(fn, _world(), port, *args)
    assert not bad, res
    skipped = [r for r in res if r and r[0].startswith("SKIP")]
    if skipped:
        pytest.skip(skipped[0][0])
    assert all(r == [] for r in res), res


def test_nvls_probes():
    import mp_cases
    _run(mp_cases.nvls_probes, 29711)


@pytest.mark.parametrize("protocol,fusion,cta_pair,steal", [("v5", "pdl", True, 1), ("v3", "pdl1", True, 1), ("v3", "none", False, 0), ("v3", "pdl", True, 0),
                                                                  ("v3r", "pdl", True, 0), ("v3r", "none", False, 0)])
def test_boundary_one_process_per_gpu(protocol, fusion, cta_pair, steal):
    import mp_cases
    port = 29712 + ["v5", "v3", "v3r"].index(protocol) * 4 + int(cta_pair) * 2 + steal
    _run(mp_cases.boundary_case, port, protocol, fusion, cta_pair, (1024, 256, 768, 1024), 2048, 8192, 2048, bool(steal))
