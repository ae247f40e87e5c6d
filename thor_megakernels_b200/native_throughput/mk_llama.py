"""``mk_llama`` module for the reference's batched ("throughput") instruction set.

The reference's loader does ``sys.path.append(mk_dir); from mk_llama import
mk_llama`` (megakernels/mk.py:5-9) and ``megakernels/demos/throughput/mk.py:7-49``
calls it with 31 positional arguments.  The reference project ships no kernel
behind that call; this module answers it with the B200 library's operator-level
executor (``mk_throughput_*`` in ``include/b200_megakernel.h``).  The handle is
created on first use and reused while the same buffers are passed; a new
``instructions`` tensor is re-validated, the same one is not.
"""
from __future__ import annotations

import sys
from pathlib import Path

_ROOT = Path(__file__).resolve().parents[2]
if str(_ROOT) not in sys.path:
    sys.path.insert(0, str(_ROOT))

from thor_megakernels_b200.batched import ThroughputExecutor  # noqa: E402

_cache: dict[tuple, ThroughputExecutor] = {}


def mk_llama(
    Bar, instructions, timings,
    qkv_weights, attn_norm_weights, o_weights, mlp_norm_weights, up_weights, gate_weights, down_weights,
    lm_head_norm_weights, lm_head_weights, k_cache, v_cache,
    rope_cos, rope_sin,
    hidden_states, rms_rope_intermediates, rms_gate_intermediates, gate_silu_intermediates, q_post_rope, attn_out,
    silu_out, rms_lm_head_intermediates, logits,
    pos_id, attn_scale, rms_norm_eps, batch_size=None,
    *, stream=None,
):
    """Run the schedule in ``instructions`` for one decode step at ``pos_id``."""
    tensors = (Bar, qkv_weights, attn_norm_weights, o_weights, mlp_norm_weights, up_weights, gate_weights, down_weights,
               lm_head_norm_weights, lm_head_weights, k_cache, v_cache, rope_cos, rope_sin, hidden_states,
               rms_rope_intermediates, rms_gate_intermediates, q_post_rope, attn_out, silu_out, rms_lm_head_intermediates,
               logits)
    key = tuple((t.data_ptr(), tuple(t.shape)) for t in tensors) + (float(attn_scale), float(rms_norm_eps))
    ex = _cache.get(key)
    if ex is None:
        if len(_cache) >= 8:
            _cache.pop(next(iter(_cache))).close()
        ex = ThroughputExecutor(
            barriers=Bar, qkv_w=qkv_weights, attn_norm_w=attn_norm_weights, o_w=o_weights, mlp_norm_w=mlp_norm_weights,
            up_w=up_weights, gate_w=gate_weights, down_w=down_weights, lm_head_norm_w=lm_head_norm_weights,
            lm_head_w=lm_head_weights, k_cache=k_cache, v_cache=v_cache, rope_cos=rope_cos, rope_sin=rope_sin,
            hidden_states=hidden_states, rms_rope_intermediates=rms_rope_intermediates,
            rms_gate_intermediates=rms_gate_intermediates, post_ln_rope_q=q_post_rope, attn_out=attn_out, silu_out=silu_out,
            rms_lm_head_intermediates=rms_lm_head_intermediates, logits=logits, attn_scale=attn_scale,
            rms_norm_eps=rms_norm_eps, batch_size=batch_size if batch_size is not None else hidden_states.shape[0],
        )
        _cache[key] = ex
    ex.set_schedule(instructions)
    ex.step(int(pos_id), stream=stream)
