"""Drop-in for the reference's compiled ``mk_llama`` extension module.

The reference loads its native kernel with ``sys.path.append(mk_dir); from
mk_llama import mk_llama`` (megakernels/mk.py:5-9) and calls it with 27
positional tensors/scalars plus ``stream=`` and ``dry_run=`` keywords
(megakernels/demos/latency/mk.py:15-49, demos/low-latency-llama/llama.cu:24-53,
include/checked_binding.cuh:17-108).  Pointing ``mk_dir`` at this directory gives
the same callable, backed by the B200 C-ABI library.  The handle behind it is
created on first use and reused while the same buffers are passed.
"""
from __future__ import annotations

import sys
from pathlib import Path

_ROOT = Path(__file__).resolve().parents[2]
if str(_ROOT) not in sys.path:
    sys.path.insert(0, str(_ROOT))

from thor_megakernels_b200.runtime import Megakernel  # noqa: E402

_cache: dict[tuple, Megakernel] = {}


def mk_llama(
    Bar, instructions, timings,
    qkv_weights, attn_norm_weights, o_weights, mlp_norm_weights, up_weights, gate_weights, down_weights,
    lm_head_norm_weights, lm_head_weights, k_cache, v_cache,
    rope_cos, rope_sin,
    hidden_states, q_post_rope, attn_out, attn_lse_intermediates, attn_out_intermediates, silu_out, logits,
    pos_id, attn_scale, rms_norm_eps, skip_attn_reduction,
    *, stream=None, dry_run=False,
):
    """Run one decode step; returns the launch-facts dict.  Raises
    ``RuntimeError`` before anything is launched when the queues do not fit the
    device or the shapes are not supported."""
    tensors = (Bar, qkv_weights, attn_norm_weights, o_weights, mlp_norm_weights, up_weights, gate_weights,
               down_weights, lm_head_norm_weights, lm_head_weights, k_cache, v_cache, rope_cos, rope_sin,
               hidden_states, q_post_rope, attn_out, attn_lse_intermediates, attn_out_intermediates, silu_out, logits)
    # addresses alone are not an identity: the allocator hands freed blocks to new tensors
    key = tuple((t.data_ptr(), tuple(t.shape)) for t in tensors) + (
        float(attn_scale), float(rms_norm_eps), bool(skip_attn_reduction))
    mk = _cache.get(key)
    if mk is None:
        if len(_cache) >= 8:  # a long-lived process that keeps re-allocating buffers
            _cache.pop(next(iter(_cache))).close()
        mk = Megakernel(
            barriers=Bar, qkv_w=qkv_weights, attn_norm_w=attn_norm_weights, o_w=o_weights,
            mlp_norm_w=mlp_norm_weights, up_w=up_weights, gate_w=gate_weights, down_w=down_weights,
            lm_head_norm_w=lm_head_norm_weights, lm_head_w=lm_head_weights, k_cache=k_cache, v_cache=v_cache,
            rope_cos=rope_cos, rope_sin=rope_sin, hidden_states=hidden_states, q_post_rope=q_post_rope,
            attn_out=attn_out, attn_lse_intermediates=attn_lse_intermediates,
            attn_out_intermediates=attn_out_intermediates, silu_out=silu_out, logits=logits,
            attn_scale=attn_scale, rms_norm_eps=rms_norm_eps, skip_attn_reduction=skip_attn_reduction,
        )
        _cache[key] = mk
    mk.set_schedule(instructions, timings)
    info = mk.query()
    if dry_run:
        return info
    mk.step(int(pos_id), stream=stream)
    return info
