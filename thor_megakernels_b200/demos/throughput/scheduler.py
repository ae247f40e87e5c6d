"""Schedule builder for the batched instruction set: buffers and the per-layer
instruction lists (reference ``megakernels/demos/throughput/scheduler.py``:
``make_globals`` :25-100, per-op splits :103-277, ``make_dag`` / ``make_dag_layer``
:280-398).

As in the reference, DAG nodes carry no explicit dependencies: ordering is by
the list (a layer's ops in opcode order, layers in order) and, on the device,
by the dependency counters.  Matmuls are cut into 128-sequence x 128-output
blocks, norms and attention are per sequence; ``batch_size`` (the model's
``extra_config.max_batch_size``) must be a multiple of 128.
"""
from __future__ import annotations

import math

import torch

from ...instructions import NoOp
from ...scheduler import DAG_Node, ScheduleBuilder
from ...utils import assert_div
from .instructions import (
    AttentionDecode,
    DownProjResidual,
    GateSilu,
    Globals,
    LM_Head,
    O_ProjResidual,
    PreAttnLayerNorm,
    PreLMHeadRMS,
    PreMLP_Norm,
    QKV_MatMulRopeAppend,
    UpMatMul,
)

MATMUL_BLOCK = 128


def make_globals(model) -> Globals:
    cfg, device, dtype = model.config, model.device, model.dtype
    bs = model.extra_config.max_batch_size
    sp = model.stacked_params

    def rows(width, dt=dtype):
        return torch.zeros((bs, width), device=device, dtype=dt)

    counters_per_row = max(cfg.num_attention_heads + 2 * cfg.num_key_value_heads,
                           assert_div(cfg.intermediate_size, MATMUL_BLOCK))
    return Globals(
        qkv_proj_weights=sp.qkv_proj, o_proj_weights=sp.o_proj, attn_ln_weights=sp.attn_ln_weight,
        mlp_ln_weights=sp.mlp_ln_weight, up_proj_weights=sp.up_proj, gate_proj_weights=sp.gate_proj,
        down_proj_weights=sp.down_proj, lm_head_norm_weights=model.lm_head.input_norm.weight,
        lm_head_weights=model.lm_head.lm_head.weight,
        k_cache=model.stacked_kv_cache[0], v_cache=model.stacked_kv_cache[1],
        rope_cos=model.model.rope_cos, rope_sin=model.model.rope_sin,
        hidden_states=rows(cfg.hidden_size),
        rms_rope_intermediates=rows(cfg.hidden_size), rms_gate_intermediates=rows(cfg.hidden_size),
        rms_lm_head_intermediates=rows(cfg.hidden_size),
        post_ln_rope_q=rows(cfg.hidden_size), attn_out=rows(cfg.hidden_size),
        silu_out=rows(cfg.intermediate_size), logits=rows(cfg.vocab_size),
        pos_id=0, attn_scale=1 / math.sqrt(cfg.head_dim), rms_norm_eps=cfg.rms_norm_eps,
        num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
        num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, hidden_size=cfg.hidden_size,
        intermediate_size=cfg.intermediate_size, vocab_size=cfg.vocab_size,
        batch_size=bs, matmul_batch_block_size=MATMUL_BLOCK, matmul_output_block_size=MATMUL_BLOCK, norm_block_size=16,
        device=device,
        # one counter row per opcode (10 > number of opcodes), per sequence
        barriers=torch.zeros([cfg.num_hidden_layers, 10, bs, counters_per_row], dtype=torch.int32, device=device),
    )


def _per_sequence(cls, globs: Globals, layer_idx: int):
    return [cls(layer_idx, b) for b in range(globs.batch_size)]


def _per_block(cls, globs: Globals, layer_idx: int, out_blocks: int):
    return [cls(layer_idx, bb, ob) for bb in range(globs.num_batch_blocks()) for ob in range(out_blocks)]


def schedule_pre_attn_norm(globs, layer_idx):
    return _per_sequence(PreAttnLayerNorm, globs, layer_idx)


def schedule_qkv_matmul_rope_append(globs, layer_idx):
    return _per_block(QKV_MatMulRopeAppend, globs, layer_idx, assert_div(globs.qkv_dim(), globs.matmul_output_block_size))


def schedule_attention_decode(globs, layer_idx):
    return [AttentionDecode(layer_idx, b, h) for b in range(globs.batch_size) for h in range(globs.num_kv_heads)]


def schedule_o_proj_residual(globs, layer_idx):
    return _per_block(O_ProjResidual, globs, layer_idx, globs.num_output_blocks())


def schedule_pre_mlp_norm(globs, layer_idx):
    return _per_sequence(PreMLP_Norm, globs, layer_idx)


def schedule_gate_silu(globs, layer_idx):
    return _per_block(GateSilu, globs, layer_idx, globs.num_intermediate_blocks())


def schedule_up_matmul(globs, layer_idx):
    return _per_block(UpMatMul, globs, layer_idx, globs.num_intermediate_blocks())


def schedule_down_proj_residual(globs, layer_idx):
    return _per_block(DownProjResidual, globs, layer_idx, globs.num_output_blocks())


def schedule_lm_head_norm(globs):
    return _per_sequence(PreLMHeadRMS, globs, 0)


def schedule_lm_head(globs):
    return [LM_Head(bb, ob) for bb in range(globs.num_batch_blocks()) for ob in range(globs.num_vocab_blocks())]


# a layer's ops in execution order, with the name that `stop_after_op` uses for each
LAYER_OPS = (
    ("attn_norm", schedule_pre_attn_norm), ("qkv", schedule_qkv_matmul_rope_append), ("attn", schedule_attention_decode),
    ("oproj", schedule_o_proj_residual), ("mlp_norm", schedule_pre_mlp_norm), ("gate", schedule_gate_silu),
    ("up", schedule_up_matmul), (None, schedule_down_proj_residual),
)


def make_dag_layer(globs: Globals, layer_idx: int, prev_layer_outputs, stop_after_op: str | None = None):
    nodes: list[DAG_Node] = []
    for name, split in LAYER_OPS:
        nodes.extend(DAG_Node(ins, prev_layer_outputs) for ins in split(globs, layer_idx))
        if name is not None and stop_after_op == name:
            return nodes, []
    assert stop_after_op is None, f"unknown stop_after_op {stop_after_op!r}"
    return nodes, []


def make_dag(globs: Globals, stop_after_op: str | None = None, layer_limit: int | None = None):
    layers = globs.num_hidden_layers if layer_limit is None else layer_limit
    nodes: list[DAG_Node] = []
    outputs: list[DAG_Node] = []
    for layer in range(layers):
        added, outputs = make_dag_layer(globs, layer, outputs, stop_after_op)
        nodes.extend(added)
    if layers == globs.num_hidden_layers:
        norm_nodes = [DAG_Node(ins, outputs) for ins in schedule_lm_head_norm(globs)]
        nodes.extend(norm_nodes)
        outputs = norm_nodes
        if stop_after_op != "lm_head_norm":
            head_nodes = [DAG_Node(ins, outputs) for ins in schedule_lm_head(globs)]
            nodes.extend(head_nodes)
            outputs = head_nodes
    return nodes, DAG_Node(NoOp(), outputs)


class ThroughputScheduleBuilder(ScheduleBuilder):
    @classmethod
    def make_globals(cls, model):
        return make_globals(model)

    @classmethod
    def make_dag(cls, globs, stop_after_op: str | None = None, layer_limit: int | None = None):
        return make_dag(globs, stop_after_op, layer_limit)
