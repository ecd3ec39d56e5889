"""Llama for vLLM with the two tensor-parallel all-reduce boundaries of every decoder layer CTA-pipelined:

  A: o_proj    -> sum over ranks + residual -> post_attention_layernorm -> gate_up_proj   (inside a layer)
  B: down_proj -> sum over ranks + residual -> next layer's input_layernorm -> its qkv_proj

Each boundary is one ``ctapp.tp4.CtappBoundary`` shared by all layers (weights are passed per call).  The RMSNorm weights
are folded into the consuming projections once, in place, after loading; the stock-path norms that remain in this forward
(layer 0, fallbacks, the final norm's input) therefore run with a weight of ones.  Tensor parallel sizes 2, 4 and 8,
pipeline parallel size 1, hidden size 8192-style models with ``hidden % 256 == 0``, eager mode.  Token counts that are not
a multiple of 128, below CTAPP_MIN_M or above CTAPP_MAX_M take the stock path.  Written for the vLLM 0.22 model API
(``LlamaModel(vllm_config=..., layer_type=...)``, ``embed_input_ids``, ``mlp.act_fn``); mirrors what the reference plugin does
for vLLM 0.30 (vllm_plugin/ctapp_vllm/model.py:26-207)."""
from __future__ import annotations

import copy
import logging
from itertools import islice

import torch
from vllm.distributed import get_pp_group, get_tensor_model_parallel_rank, get_tensor_model_parallel_world_size, get_tp_group
from vllm.model_executor.models.llama import LlamaDecoderLayer, LlamaForCausalLM, LlamaModel

from . import knobs

logger = logging.getLogger("ctapp_vllm")


@torch.no_grad()
def fold_norm_weights(layers):
    """qkv_proj.weight *= input_layernorm.weight and gate_up_proj.weight *= post_attention_layernorm.weight (columns), fp32
    arithmetic, bf16 storage, in place, 2048 rows at a time."""
    for layer in layers:
        for W, gamma in ((layer.self_attn.qkv_proj.weight, layer.input_layernorm.weight),
                         (layer.mlp.gate_up_proj.weight, layer.post_attention_layernorm.weight)):
            g32 = gamma.float()[None, :]
            for r0 in range(0, W.shape[0], 2048):
                W[r0:r0 + 2048] = (W[r0:r0 + 2048].float() * g32).to(W.dtype)


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm()).item()


class CtappLlamaModel(LlamaModel):
    def __init__(self, *, vllm_config, prefix="", layer_type=LlamaDecoderLayer):
        super().__init__(vllm_config=vllm_config, prefix=prefix, layer_type=layer_type)
        self._k = knobs()
        t = get_tensor_model_parallel_world_size()
        self._usable = (t in (2, 4, 8) and get_pp_group().world_size == 1 and self.config.hidden_size % 256 == 0)
        self._pool_a = self._pool_b = None
        self._folded = False
        self._ones = None
        self._seen = set()
        if not self._usable:
            logger.warning("ctapp_vllm: boundaries disabled for this configuration (needs TP 2/4/8, PP 1, hidden %% 256 == 0)")

    # ---- one-time set-up, after the weights are loaded
    def _own_layers(self):
        return list(islice(self.layers, self.start_layer, self.end_layer))

    def _fold(self):
        layers = self._own_layers()
        fold_norm_weights(layers)
        if self._ones is None:
            ones = copy.deepcopy(layers[0].input_layernorm)
            for p in ones.parameters():
                p.requires_grad_(False)
            object.__setattr__(self, "_ones", ones)        # not a checkpoint weight: keep it out of the module tree
        self._ones.weight.fill_(1.0)
        self._folded = True

    def _refold(self):
        """Call after re-initialising weights: the next forward folds the norm weights again."""
        self._folded = False

    def _setup(self, device):
        from ctapp.tp4 import CtappBoundaryPool
        k = self._k
        self._fold()
        l0 = self._own_layers()[0]
        hidden = self.config.hidden_size
        rank, t = get_tensor_model_parallel_rank(), get_tensor_model_parallel_world_size()
        group = get_tp_group().device_group.group_name
        common = dict(R=k["R"], min_M=k["min_M"], protocol=k["proto"], max_M=k["max_M"], fusion=k["fusion"], n1=hidden,
                      eps=self.config.rms_norm_eps)
        self._pool_b = CtappBoundaryPool(l0.mlp.down_proj.weight.shape[1], l0.self_attn.qkv_proj.weight.shape[0], rank, t, group, device,
                                         qkv_raster=k["b_raster"], qkv_swizzle=k["b_swizzle"], qkv_tile=k["qkv_tile"], steal=k["steal_b"], **common)
        self._pool_a = CtappBoundaryPool(l0.self_attn.o_proj.weight.shape[1], l0.mlp.gate_up_proj.weight.shape[0], rank, t, group, device,
                                         qkv_raster=k["a_raster"], qkv_swizzle=k["a_swizzle"], qkv_tile=256, down_tail=hidden // 256,
                                         steal=k["steal_a"], **common)
        if k["cksum"] and rank == 0:
            w = l0.mlp.down_proj.weight.float()
            logger.warning("CTAPP_CKSUM layers[0].down_proj.weight rank0 shape=%s sum=%.6e abssum=%.6e", tuple(w.shape), w.sum().item(), w.abs().sum().item())
        logger.warning("ctapp_vllm rank %d: set-up done (%s)", rank, {kk: v for kk, v in k.items() if kk != "enabled"})

    def _boundaries(self, M):
        """(boundary A or None, boundary B or None) for this token count; creation is collective, so every rank quiesces
        its GPU and meets the others around it."""
        k = self._k
        out = []
        for pool, wanted in ((self._pool_a, k["boundary"] in ("both", "oproj")), (self._pool_b, k["boundary"] in ("both", "down"))):
            if not wanted:
                out.append(None)
                continue
            creating = not pool._inst and pool.supports(M)
            if creating:
                torch.cuda.synchronize()
                get_tp_group().barrier()
            out.append(pool.get(M))
            if creating:
                torch.cuda.synchronize()
                get_tp_group().barrier()
        return out

    def forward(self, input_ids, positions, intermediate_tensors, inputs_embeds=None, **extra_layer_kwargs):
        if not self._usable:
            return super().forward(input_ids, positions, intermediate_tensors, inputs_embeds, **extra_layer_kwargs)
        x = inputs_embeds if inputs_embeds is not None else self.embed_input_ids(input_ids)
        M = x.shape[0]
        if self._pool_a is None:
            self._setup(x.device)
        elif not self._folded:
            self._fold()
        ones, k = self._ones, self._k
        ba, bb = self._boundaries(M)
        rank = get_tensor_model_parallel_rank()
        if rank == 0 and (M not in self._seen or k["log_M"]):
            self._seen.add(M)
            logger.warning("ctapp_vllm forward M=%d -> A:%s B:%s", M, ba is not None, bb is not None)
        layers = self._own_layers()
        residual, qkv = None, None
        for i, layer in enumerate(layers):
            attn, mlp = layer.self_attn, layer.mlp
            nxt = layers[i + 1] if i + 1 < len(layers) else None
            if qkv is None:                                   # stock norm + QKV (layer 0, or the previous boundary B fell back)
                if residual is None:
                    residual, h = x, ones(x)
                else:
                    h, residual = ones(x, residual)
                qkv, _ = attn.qkv_proj(h)
            q, kk, v = qkv.split([attn.q_size, attn.kv_size, attn.kv_size], dim=-1)
            q, kk = attn.rotary_emb(positions, q, kk)
            a = attn.attn(q, kk, v)
            if ba is not None:
                a = a if a.is_contiguous() else a.contiguous()
                ref = None
                if k["check"]:                                # stock result first; same collectives on every rank
                    y, _ = attn.o_proj(a)
                    y, r2 = ones(y, residual.clone())
                    ref = (mlp.gate_up_proj(y)[0], r2)
                g = ba.forward(a, residual, Wd=attn.o_proj.weight, Wq=mlp.gate_up_proj.weight)
                residual = ba.x()
                if ref is not None and rank == 0:
                    logger.warning("CTAPP_CHECK M=%d layer %d A: out rel %.3e  x rel %.3e", M, i, _rel(g, ref[0]), _rel(residual, ref[1]))
            else:
                y, _ = attn.o_proj(a)                          # stock all-reduce inside
                y, residual = ones(y, residual)
                g, _ = mlp.gate_up_proj(y)
            h_r = mlp.act_fn(g)
            if bb is not None and nxt is not None:
                ref = None
                if k["check"]:
                    y, _ = mlp.down_proj(h_r)
                    y, r2 = ones(y, residual.clone())
                    ref = (nxt.self_attn.qkv_proj(y)[0], r2)
                qkv = bb.forward(h_r, residual, Wd=mlp.down_proj.weight, Wq=nxt.self_attn.qkv_proj.weight)
                residual = bb.x()
                x = None
                if ref is not None and rank == 0:
                    logger.warning("CTAPP_CHECK M=%d layer %d->%d B: out rel %.3e  x rel %.3e", M, i, i + 1, _rel(qkv, ref[0]), _rel(residual, ref[1]))
            else:
                x, _ = mlp.down_proj(h_r)
                qkv = None
        out, _ = self.norm(x, residual)
        return out


class CtappLlamaForCausalLM(LlamaForCausalLM):
    def _init_model(self, vllm_config, prefix="", layer_type=LlamaDecoderLayer):
        return CtappLlamaModel(vllm_config=vllm_config, prefix=prefix, layer_type=layer_type)
