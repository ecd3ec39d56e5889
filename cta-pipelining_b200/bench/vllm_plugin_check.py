"""Runs the vLLM plugin's model (``ctapp_vllm.model.CtappLlamaForCausalLM``) inside vLLM's own distributed environment,
without the serving engine around it, and compares it with the stock model on the same dummy weights and token ids.

    python cta-pipelining_b200/bench/vllm_plugin_check.py [--tp 2] [--layers 2] [--tokens 4096] [--out FILE]

One process per GPU (spawned here).  Every rank
  1. builds vLLM's configuration for a Llama-70B-shaped model with ``--layers`` layers from a generated ``config.json``
     (``load_format="dummy"``: seeded random weights, no checkpoint; no tokenizer),
  2. brings up vLLM's process groups itself (``init_distributed_environment`` + ``initialize_model_parallel``),
  3. loads the stock ``LlamaForCausalLM`` through vLLM's model loader, runs one forward over ``--tokens`` seeded token ids and
     keeps the hidden states and the top-1 / top-20 tokens of every position,
  4. registers the plugin (``CTAPP_VLLM=1``, ``ctapp_vllm.register()``), loads the model again -- the registry now resolves the
     architecture to the plugin's class, the dummy loader draws the same weights -- runs the same forward with
     ``CTAPP_CHECK=1`` (per-layer relative error of both boundaries against the stock path, logged by the plugin) and compares.
Forwards run the way vLLM's profiling run does (no attention metadata: the attention kernels are skipped and their output
buffer is passed on), which leaves the projections, norms, activations and both tensor-parallel boundaries of every layer in
place: what this check is about.  Mirrors reference bench/vllm_ctapp_check.py:44-71 (per-layer error lines, top-1 / top-20
agreement); that script goes through ``vllm.LLM``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
for p in (PKG, os.path.join(PKG, "vllm_plugin")):
    if p not in sys.path:
        sys.path.insert(0, p)


def llama_config(layers, hidden=8192, ffn=28672, heads=64, kv_heads=8, vocab=128256):
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": hidden, "intermediate_size": ffn,
            "num_attention_heads": heads, "num_key_value_heads": kv_heads, "num_hidden_layers": layers, "vocab_size": vocab,
            "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 16384, "hidden_act": "silu",
            "tie_word_embeddings": False, "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2}


def worker(rank, world, port, cfg_dir, tokens, results):
    import logging
    import torch
    os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0", "VLLM_LOGGING_LEVEL": "WARNING"})
    torch.cuda.set_device(rank)
    out = {"rank": rank}
    try:
        from vllm.config import set_current_vllm_config
        from vllm.distributed.parallel_state import init_distributed_environment, initialize_model_parallel
        from vllm.engine.arg_utils import EngineArgs
        from vllm.forward_context import set_forward_context
        from vllm.model_executor.model_loader import get_model

        args = EngineArgs(model=cfg_dir, load_format="dummy", tensor_parallel_size=world, enforce_eager=True, skip_tokenizer_init=True,
                          max_model_len=max(8192, tokens), dtype="bfloat16", seed=0)
        vcfg = args.create_engine_config()
        checks = []

        class Catch(logging.Handler):
            def emit(self, record):
                msg = record.getMessage()
                if msg.startswith("CTAPP_CHECK"):
                    checks.append(msg)
        logging.getLogger("ctapp_vllm").addHandler(Catch())

        g = torch.Generator().manual_seed(0)
        ids = torch.randint(1000, 50000, (tokens,), generator=g).cuda()
        pos = torch.arange(tokens, device="cuda")

        def run(model):
            with torch.no_grad(), set_forward_context(None, vcfg, num_tokens=tokens):
                h = model(ids, pos)
                logits = model.compute_logits(h)
            torch.cuda.synchronize()
            return h.float().cpu(), logits.float().topk(20, dim=-1).indices.cpu()

        with set_current_vllm_config(vcfg):
            init_distributed_environment(world, rank, f"tcp://127.0.0.1:{port}", rank, "nccl")
            initialize_model_parallel(world)
            t0 = time.time()
            stock = get_model(vllm_config=vcfg)
            out["stock_class"] = type(stock).__name__
            h0, top0 = run(stock)
            del stock
            torch.cuda.empty_cache()
            vcfg.compilation_config.static_forward_context.clear()      # the attention layers register themselves by name: start afresh
            os.environ.update({"CTAPP_VLLM": "1", "CTAPP_CHECK": "1", "CTAPP_MIN_M": "128"})
            import ctapp_vllm
            ctapp_vllm.register()
            # vLLM remembers which class an architecture resolved to; a serving process registers the plugin before anything
            # is resolved, this process resolved the stock class a moment ago
            from vllm.model_executor.model_loader import utils as loader_utils
            getattr(loader_utils, "_MODEL_ARCH_BY_HASH", {}).clear()
            ours = get_model(vllm_config=vcfg)
            out["plugin_class"] = type(ours).__name__
            h1, top1 = run(ours)                 # first forward: folds the norm weights, creates both boundaries (collective)
            h2, _ = run(ours)                    # and again on the warm instance
            out["seconds"] = round(time.time() - t0, 1)
        rel = lambda a, b: float((a - b).norm() / b.norm())  # noqa: E731
        out.update(hidden_rel=rel(h1, h0), hidden_rel_second_forward=rel(h2, h0), nan=bool(torch.isnan(h1).any()),
                   top1_agree=float((top1[:, 0] == top0[:, 0]).float().mean()),
                   top1_in_stock_top20=float((top1[:, :1] == top0).any(-1).float().mean()),
                   checks=checks[: 4 * 8], n_checks=len(checks), ok=True)
    except BaseException as e:  # noqa: BLE001
        import traceback
        out.update(ok=False, error=repr(e)[:500], trace=traceback.format_exc()[-3000:])
    results.put(out)
    try:
        import torch
        torch.cuda.synchronize()
    except Exception:  # noqa: BLE001
        pass
    time.sleep(2.0)
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--port", type=int, default=29811)
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    import torch.multiprocessing as mp
    cfg_dir = tempfile.mkdtemp(prefix="llama70b_shape_")
    json.dump(llama_config(a.layers), open(os.path.join(cfg_dir, "config.json"), "w"))
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, a.tp, a.port, cfg_dir, a.tokens, q)) for r in range(a.tp)]
    for p in procs:
        p.start()
    res = []
    deadline = time.time() + 900
    while len(res) < a.tp and time.time() < deadline and (any(p.is_alive() for p in procs) or not q.empty()):
        try:
            res.append(q.get(timeout=2))
        except Exception:  # noqa: BLE001
            pass
    for p in procs:
        p.join(timeout=30)
    res.sort(key=lambda r: r["rank"])
    text = json.dumps({"tp": a.tp, "layers": a.layers, "tokens": a.tokens, "ranks": res}, indent=1)
    print(text)
    if a.out:
        open(a.out, "w").write(text)
    sys.exit(0 if len(res) == a.tp and all(r.get("ok") for r in res) else 1)


if __name__ == "__main__":
    main()
