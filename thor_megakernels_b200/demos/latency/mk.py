"""Marshals a latency ``Globals`` into the native step call
(reference ``megakernels/demos/latency/mk.py:8-54``): same 27 positional
arguments in the same order, KV caches flattened to ``[(L B), T, Hkv, D]``,
launch on the caller's current CUDA stream."""
from __future__ import annotations

import torch

from ...mk import MK_Interpreter
from .instructions import Globals


def interpret_with_mk(globs: Globals, mk_func):
    k4 = globs.k_cache.flatten(0, 1)
    v4 = globs.v_cache.flatten(0, 1)
    return mk_func(
        globs.barriers, globs.instructions, globs.timings,
        globs.qkv_proj_weights, globs.attn_ln_weights, globs.o_proj_weights, globs.mlp_ln_weights,
        globs.up_proj_weights, globs.gate_proj_weights, globs.down_proj_weights,
        globs.lm_head_norm_weights.data, globs.lm_head_weights.data, k4, v4,
        globs.rope_cos, globs.rope_sin,
        globs.hidden_states, globs.post_ln_rope_q, globs.attn_out,
        globs.attn_lse_intermediates, globs.attn_out_intermediates, globs.silu_out, globs.logits,
        globs.pos_id, globs.attn_scale, globs.rms_norm_eps, globs.skip_attn_reduction,
        stream=torch.cuda.current_stream(),
    )


class LatencyMK_Interpreter(MK_Interpreter):
    def interpret(self, globs: Globals):
        return interpret_with_mk(globs, self.mk_func)
