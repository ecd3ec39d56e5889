"""The standalone Llama-70B-shape prefill harness (``cta-pipelining_b200/bench/llama_prefill.py``) on a two-layer slice: both
boundaries of every layer through ``CtappBoundary`` against the stock path (cuBLAS + all-reduce + fused add-RMSNorm) on the same
weights.  Mirrors what reference bench/vllm_ctapp_check.py:44-71 checks on a 4-layer model: per-layer boundary errors and the
final hidden state."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPT = os.path.join(ROOT, "cta-pipelining_b200", "bench", "llama_prefill.py")


def _check(out):
    lines = [l for l in out.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out[-2000:]
    d = json.loads(lines[0])
    assert d["stock_ms"] > 0 and d["pipelined_ms"] > 0
    # relative Frobenius-norm difference per boundary, bounded as the reference bounds its own end-to-end test (x < 1e-2, out < 2e-2,
    # tests/test_tp4.py:110-111); measured 2.4e-3 to 4.6e-3
    assert d["per_layer_check"], d
    for c in d["per_layer_check"]:
        assert c["out_rel"] < 2e-2 and c["x_rel"] < 1e-2, c
    assert d["final_hidden_rel_vs_stock"] < 3e-2, d["final_hidden_rel_vs_stock"]
    return d


@pytest.mark.parametrize("act", ["kernel", "fused"])
def test_two_layer_prefill_one_gpu(act):
    """One rank (nothing to exchange, every kernel of a boundary on one stream): the harness runs and both paths agree."""
    r = subprocess.run([sys.executable, SCRIPT, "--layers", "2", "--tokens", "512", "--iters", "1", "--check", "2", "--fusion", "serial", "--act", act],
                       capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-3000:]
    _check(r.stdout)


@pytest.mark.multigpu(2)
def test_two_layer_prefill_two_gpus():
    """TP2, producer / reducer / consumer overlapping within and across the GPUs (``fusion="pdl"``)."""
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29791", SCRIPT, "--layers", "2", "--tokens", "1024", "--iters", "1", "--check", "2"],
                       capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-3000:]
    _check(r.stdout)
