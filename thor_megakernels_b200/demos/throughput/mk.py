"""Marshals a batched-instruction-set ``Globals`` into the native step call
(reference ``megakernels/demos/throughput/mk.py:7-49``): the same 31 positional
arguments in the same order (``silu_out`` appears twice there, once in the
place of the commented-out ``gate_silu_intermediates``), KV caches flattened to
``[(L B), T, Hkv, D]``."""
from __future__ import annotations

from ...mk import THROUGHPUT_MK_DIR, MK_Interpreter
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
        globs.hidden_states, globs.rms_rope_intermediates, globs.rms_gate_intermediates,
        globs.silu_out, globs.post_ln_rope_q, globs.attn_out, globs.silu_out,
        globs.rms_lm_head_intermediates, globs.logits,
        globs.pos_id, globs.attn_scale, globs.rms_norm_eps, globs.batch_size,
    )


class ThroughputMK_Interpreter(MK_Interpreter):
    default_mk_dir = THROUGHPUT_MK_DIR

    def interpret(self, globs: Globals):
        return interpret_with_mk(globs, self.mk_func)
