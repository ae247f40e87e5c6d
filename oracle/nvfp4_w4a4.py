"""TEST INFRASTRUCTURE ONLY - CPU oracle for one decode step of a Llama model
whose linears run NVFP4 x NVFP4 (weights quantised once, activations quantised
on the fly), the numerics of the reference's native FP4 path:

* activation quantiser ``include/ops/nvfp4_linear.cuh:174-237``: the bf16 input
  of a linear (after RMSNorm with two bf16 roundings, or after the SiLU-gate
  product with one) is divided by its tensor scale, every 16 consecutive values
  get ``scale = e4m3(max(amax / 6, 2^-9))`` and codes ``e2m1(v / scale)`` - the
  same arithmetic as the weight quantiser (``oracle/nvfp4.py``);
* linear ``:52-173``: exact products of the decoded operands, accumulated
  (float64 here), times both tensor scales, one bf16 rounding (``:147``);
* residual adds in bf16; attention, rotary embedding and KV append as in the
  bf16 interpreter (``oracle/pyvm.py``).

The weight plan is the one of ``oracle/nvfp4_model.py``.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from oracle import nvfp4
from oracle.nvfp4_model import QuantMatrix
from oracle.pyvm import rms_norm
from thor_megakernels_b200.llama import apply_rotary_pos_emb_interleaved


def quantize_activations(x_bf16: torch.Tensor, tensor_scale: float = 1.0) -> torch.Tensor:
    """bf16 vector -> what the tensor core sees after NVFP4 quantisation, as float64."""
    x = x_bf16.float().numpy().reshape(1, -1)
    packed, scales, decoded = nvfp4.quantize(x, np.float32(tensor_scale))
    return torch.from_numpy(decoded.astype(np.float64)).view(-1)


def linear_a4(x_bf16: torch.Tensor, q: QuantMatrix, tensor_scale: float = 1.0) -> torch.Tensor:
    return (q.dequant.double() @ quantize_activations(x_bf16, tensor_scale)).float().bfloat16()


@torch.no_grad()
def decode_step(model, layers, head, hidden_in: torch.Tensor, pos_id: int, cache_slot: int = 0, activation_scale: float = 1.0):
    """One decode token of one sequence (cache slot ``cache_slot``).  Returns
    (hidden, logits, dict of the last layer's intermediate buffers)."""
    cfg = model.config
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    group, scale = hq // hkv, 1 / math.sqrt(d)
    hidden = hidden_in.clone()
    sp = model.stacked_params
    k_cache, v_cache = model.stacked_kv_cache
    cos, sin = model.model.rope_cos[pos_id], model.model.rope_sin[pos_id]
    lin = lambda x, q: linear_a4(x, q, activation_scale)
    last = {}
    for i, ql in enumerate(layers):
        x = rms_norm(hidden, sp.attn_ln_weight[i], cfg.rms_norm_eps)
        qkv = lin(x, ql.qkv)
        q, k, v = qkv[: hq * d].view(hq, d), qkv[hq * d : (hq + hkv) * d].view(hkv, d), qkv[(hq + hkv) * d :].view(hkv, d)
        q_r, k_r = apply_rotary_pos_emb_interleaved(q, k, cos, sin, unsqueeze_dim=0)
        q_r, k_r = q_r.to(qkv.dtype), k_r.to(qkv.dtype)
        k_cache[i, cache_slot, pos_id] = k_r
        v_cache[i, cache_slot, pos_id] = v
        attn = torch.empty(hq, d, dtype=torch.float32)
        for kvh in range(hkv):
            kk = k_cache[i, cache_slot, : pos_id + 1, kvh].float()
            vv = v_cache[i, cache_slot, : pos_id + 1, kvh].float()
            qq = q_r[kvh * group : (kvh + 1) * group].float()
            attn[kvh * group : (kvh + 1) * group] = torch.softmax((qq @ kk.T) * scale, dim=-1) @ vv
        attn_bf = attn.bfloat16().view(-1)
        hidden = hidden + lin(attn_bf, ql.o)
        x2 = rms_norm(hidden, sp.mlp_ln_weight[i], cfg.rms_norm_eps)
        up, gate = lin(x2, ql.up), lin(x2, ql.gate)
        prod = (F.silu(gate.float()) * up.float()).bfloat16()
        hidden = hidden + lin(prod, ql.down)
        last = dict(q=q_r.reshape(-1), attn_out=attn_bf, silu_out=prod)
    logits = lin(rms_norm(hidden, model.lm_head.input_norm.weight, cfg.rms_norm_eps), head)
    return hidden, logits, last
