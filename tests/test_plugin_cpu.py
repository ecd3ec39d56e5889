"""The vLLM plugin's host-side pieces that need neither a GPU nor the serving engine: knob parsing, the off switch, and the
in-place folding of the norm weights (against the library's ``fold_gamma``)."""
import os
import sys
import types

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "cta-pipelining_b200", "vllm_plugin"))


def test_knobs_defaults_and_validation():
    import ctapp_vllm
    k = ctapp_vllm.knobs({})
    assert k == {"enabled": False, "boundary": "both", "proto": "v5", "fusion": "pdl", "qkv_tile": 256, "max_M": 8192, "min_M": 512,
                 "R": None, "check": False, "log_M": False, "cksum": False, "steal_a": True, "steal_b": False,
                 "a_raster": 3, "a_swizzle": 4, "b_raster": 2, "b_swizzle": 1}
    k = ctapp_vllm.knobs({"CTAPP_STEAL": "0", "CTAPP_FUSION": "pdl1", "CTAPP_A_RASTER": "2", "CTAPP_B_SWIZZLE": "2", "CTAPP_CKSUM": "1"})
    assert (k["steal_a"], k["steal_b"], k["fusion"], k["a_raster"], k["b_swizzle"], k["cksum"]) == (False, False, "pdl1", 2, 2, True)
    assert ctapp_vllm.knobs({"CTAPP_STEAL": "1"})["steal_b"]
    k = ctapp_vllm.knobs({"CTAPP_VLLM": "1", "CTAPP_BOUNDARY": "down", "CTAPP_PROTO": "v3", "CTAPP_FUSION": "none", "CTAPP_QKV_TILE": "128",
                          "CTAPP_MAX_M": "16384", "CTAPP_MIN_M": "256", "CTAPP_R": "8", "CTAPP_CHECK": "1"})
    assert k["enabled"] and k["boundary"] == "down" and k["proto"] == "v3" and k["fusion"] == "none" and k["qkv_tile"] == 128
    assert k["max_M"] == 16384 and k["min_M"] == 256 and k["R"] == 8 and k["check"]
    for bad in ({"CTAPP_BOUNDARY": "up"}, {"CTAPP_PROTO": "v9"}, {"CTAPP_FUSION": "warp"}, {"CTAPP_QKV_TILE": "64"}):
        with pytest.raises(ValueError):
            ctapp_vllm.knobs(bad)


def test_register_is_a_no_op_when_switched_off(monkeypatch):
    import ctapp_vllm
    monkeypatch.delenv("CTAPP_VLLM", raising=False)
    before = set(sys.modules)
    ctapp_vllm.register()
    assert not any(m.startswith("vllm") for m in set(sys.modules) - before), "the serving engine must not be imported when the plugin is off"


def test_fold_norm_weights_matches_fold_gamma():
    from ctapp.tp4 import fold_gamma
    src = open(os.path.join(ROOT, "cta-pipelining_b200", "vllm_plugin", "ctapp_vllm", "model.py")).read()
    # take the pure helper out of the module (its imports need the serving engine)
    start = src.index("@torch.no_grad()\ndef fold_norm_weights")
    end = src.index("def _rel(")
    ns = {"torch": torch}
    exec(src[start:end], ns)
    g = torch.Generator().manual_seed(0)
    def lin(rows, cols):
        return types.SimpleNamespace(weight=(torch.randn(rows, cols, generator=g) * cols ** -0.5).to(torch.bfloat16))
    def norm(n):
        return types.SimpleNamespace(weight=(0.5 + torch.rand(n, generator=g)).to(torch.bfloat16))
    layers = [types.SimpleNamespace(self_attn=types.SimpleNamespace(qkv_proj=lin(2304, 512)), mlp=types.SimpleNamespace(gate_up_proj=lin(4100, 512)),
                                    input_layernorm=norm(512), post_attention_layernorm=norm(512)) for _ in range(2)]
    want = [(fold_gamma(l.self_attn.qkv_proj.weight, l.input_layernorm.weight), fold_gamma(l.mlp.gate_up_proj.weight, l.post_attention_layernorm.weight))
            for l in layers]
    ns["fold_norm_weights"](layers)
    for l, (wq, wg) in zip(layers, want):
        assert torch.equal(l.self_attn.qkv_proj.weight, wq) and torch.equal(l.mlp.gate_up_proj.weight, wg)
