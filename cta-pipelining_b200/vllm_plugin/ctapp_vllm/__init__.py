"""vLLM general plugin (entry point group ``vllm.general_plugins``, name ``ctapp``).  Off unless CTAPP_VLLM=1; when on, the
Llama architecture is served by ``ctapp_vllm.model.CtappLlamaForCausalLM``, whose tensor-parallel all-reduce boundaries run
through ``ctapp.tp4.CtappBoundary``.  Same switch and knobs as the reference plugin (vllm_plugin/ctapp_vllm/__init__.py:10-24,
model.py:31-38,60-70)."""
import logging
import os
import sys

logger = logging.getLogger("ctapp_vllm")
_announced = False


def knobs(env=None):
    """The CTAPP_* environment knobs as a dict (pure function of ``env``; defaults as in the reference's README table)."""
    e = os.environ if env is None else env
    mode = e.get("CTAPP_BOUNDARY", "both")
    proto = e.get("CTAPP_PROTO", "v5")
    fusion = e.get("CTAPP_FUSION", "pdl")
    if mode not in ("both", "down", "oproj"):
        raise ValueError(f"CTAPP_BOUNDARY={mode!r}: expected both | down | oproj")
    if proto not in ("v3", "v3r", "v5"):
        raise ValueError(f"CTAPP_PROTO={proto!r}: expected v3 | v3r | v5")
    if fusion not in ("none", "pdl", "pdl1", "role"):
        raise ValueError(f"CTAPP_FUSION={fusion!r}: this build has none | pdl | pdl1 | role")
    tile = int(e.get("CTAPP_QKV_TILE", "256"))
    if tile not in (128, 256):
        raise ValueError(f"CTAPP_QKV_TILE={tile}: expected 128 | 256")
    return {"enabled": e.get("CTAPP_VLLM", "0") == "1", "boundary": mode, "proto": proto, "fusion": fusion, "qkv_tile": tile,
            "max_M": int(e.get("CTAPP_MAX_M", "8192")), "min_M": int(e.get("CTAPP_MIN_M", "512")),
            "R": int(e["CTAPP_R"]) if e.get("CTAPP_R") else None, "check": e.get("CTAPP_CHECK", "0") == "1",
            "log_M": e.get("CTAPP_LOG_M", "0") == "1", "cksum": e.get("CTAPP_CKSUM", "0") == "1",
            # CTAPP_STEAL unset: boundary A steals, B does not (the reference's default); set: both boundaries follow it
            "steal_a": e.get("CTAPP_STEAL", "1") == "1", "steal_b": e.get("CTAPP_STEAL", "0") == "1",
            # consumer tile orders (raster 2 = n fastest, 3 = groups of `swizzle` tile rows, else m fastest); the defaults are
            # the orders measured best with this library's kernels, not the reference's CUTLASS raster numbers
            "a_raster": int(e.get("CTAPP_A_RASTER", "3")), "a_swizzle": int(e.get("CTAPP_A_SWIZZLE", "4")),
            "b_raster": int(e.get("CTAPP_B_RASTER", "2")), "b_swizzle": int(e.get("CTAPP_B_SWIZZLE", "1"))}


def register():
    global _announced
    on = os.environ.get("CTAPP_VLLM", "0") == "1"
    if not _announced:
        _announced = True
        logger.warning("ctapp_vllm plugin loaded in pid %d: CTAPP_VLLM=%s -> %s", os.getpid(), os.environ.get("CTAPP_VLLM", "0"),
                       "CTA-pipelined boundaries ENABLED" if on else "stock model")
    if not on:
        return
    pkg = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", ".."))    # the directory that holds the ctapp package
    if pkg not in sys.path:
        sys.path.insert(0, pkg)
    from vllm.model_executor.models.registry import ModelRegistry
    ModelRegistry.register_model("LlamaForCausalLM", "ctapp_vllm.model:CtappLlamaForCausalLM")
