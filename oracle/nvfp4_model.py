"""TEST INFRASTRUCTURE ONLY - CPU oracle for one decode step of a Llama model
whose linear layers are NVFP4 weight-only (bf16 activations and KV cache).

Follows the reference's quantised-model oracle
``tools/analysis/nvfp4/model_reference.py:39-61``:

* every linear is ``F.linear(x.float(), dequantised_fp32).bfloat16()`` - fp32
  accumulation over the whole input width, one bf16 rounding;
* the MLP product is ``(silu(gate.float()) * up.float()).bfloat16()`` - one
  rounding, not the two of the bf16 interpreter;
* residual adds are plain bf16 adds of the rounded linear output.

and the weight plan of ``experimental/native_fp4_vm/model.cu:112-126`` /
``tools/analysis/nvfp4/model_bench.py:43-55``: per layer qkv, o, up and gate
concatenated (quantised as ONE matrix, so they share a tensor scale), down; plus
the LM head.  RMSNorm, rotary embedding, KV append and attention are those of the
bf16 interpreter (``oracle/pyvm.py``): fp32 softmax attention over the cache.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F

from oracle import nvfp4
from oracle.pyvm import rms_norm
from thor_megakernels_b200.llama import apply_rotary_pos_emb_interleaved


@dataclass
class QuantMatrix:
    packed: np.ndarray       # uint8 [rows, k/2]
    scales: np.ndarray       # uint8 [rows, k/16]
    tensor_scale: np.float32
    dequant: torch.Tensor    # fp32 [rows, k]


def quantize_matrix(w_bf16: torch.Tensor, tensor_scale=None) -> QuantMatrix:
    w = w_bf16.float().numpy()
    ts = nvfp4.tensor_scale_for(np.abs(w).max()) if tensor_scale is None else np.float32(tensor_scale)
    packed, scales, decoded = nvfp4.quantize(w, ts)
    return QuantMatrix(packed, scales, ts, torch.from_numpy(decoded))


@dataclass
class QuantLayer:
    qkv: QuantMatrix
    o: QuantMatrix
    up: QuantMatrix
    gate: QuantMatrix
    down: QuantMatrix


def quantize_model(model):
    """Quantise every linear of a finalised model container.  up and gate take the
    tensor scale of their concatenation."""
    sp = model.stacked_params
    layers = []
    for i in range(model.config.num_hidden_layers):
        ug_scale = nvfp4.tensor_scale_for(max(sp.up_proj[i].abs().max().item(), sp.gate_proj[i].abs().max().item()))
        layers.append(QuantLayer(
            qkv=quantize_matrix(sp.qkv_proj[i]), o=quantize_matrix(sp.o_proj[i]),
            up=quantize_matrix(sp.up_proj[i], ug_scale), gate=quantize_matrix(sp.gate_proj[i], ug_scale),
            down=quantize_matrix(sp.down_proj[i]),
        ))
    head = quantize_matrix(model.lm_head.lm_head.weight.data)
    return layers, head


def _linear(x_bf16: torch.Tensor, q: QuantMatrix) -> torch.Tensor:
    return F.linear(x_bf16.float(), q.dequant).bfloat16()


@torch.no_grad()
def decode_step(model, layers, head, hidden_in: torch.Tensor, pos_id: int):
    """One decode token.  ``hidden_in`` is the embedded input (bf16 [hidden]).
    Updates the model's KV cache at ``pos_id``; returns (hidden, logits, per-layer
    dict of intermediate buffers of the last layer)."""
    cfg = model.config
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    group = hq // hkv
    scale = 1 / math.sqrt(d)
    hidden = hidden_in.clone()
    sp = model.stacked_params
    k_cache, v_cache = model.stacked_kv_cache
    cos, sin = model.model.rope_cos[pos_id], model.model.rope_sin[pos_id]
    last = {}
    for i, ql in enumerate(layers):
        x = rms_norm(hidden, sp.attn_ln_weight[i], cfg.rms_norm_eps)
        qkv = _linear(x, ql.qkv)
        q, k, v = qkv[: hq * d].view(hq, d), qkv[hq * d : (hq + hkv) * d].view(hkv, d), qkv[(hq + hkv) * d :].view(hkv, d)
        q_r, k_r = apply_rotary_pos_emb_interleaved(q, k, cos, sin, unsqueeze_dim=0)
        q_r, k_r = q_r.to(qkv.dtype), k_r.to(qkv.dtype)
        k_cache[i, 0, pos_id] = k_r
        v_cache[i, 0, pos_id] = v
        attn = torch.empty(hq, d, dtype=torch.float32)
        for kvh in range(hkv):
            kk = k_cache[i, 0, : pos_id + 1, kvh].float()
            vv = v_cache[i, 0, : pos_id + 1, kvh].float()
            qq = q_r[kvh * group : (kvh + 1) * group].float()
            probs = torch.softmax((qq @ kk.T) * scale, dim=-1)
            attn[kvh * group : (kvh + 1) * group] = probs @ vv
        attn_bf = attn.bfloat16().view(-1)
        hidden = hidden + _linear(attn_bf, ql.o)
        x2 = rms_norm(hidden, sp.mlp_ln_weight[i], cfg.rms_norm_eps)
        up, gate = _linear(x2, ql.up), _linear(x2, ql.gate)
        prod = (F.silu(gate.float()) * up.float()).bfloat16()
        hidden = hidden + _linear(prod, ql.down)
        last = dict(q=q_r.reshape(-1), attn_out=attn_bf, silu_out=prod)
    logits = _linear(rms_norm(hidden, model.lm_head.input_norm.weight, cfg.rms_norm_eps), head)
    return hidden, logits, last
