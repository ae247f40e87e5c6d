"""TEST INFRASTRUCTURE ONLY - PyTorch (CPU) interpreter of the batched
("throughput") instruction set, restating the reference's oracle

    megakernels/demos/throughput/python_vm.py:26-465   (per-opcode solvers)
    megakernels/python_vm.py:83-95                     (interpreter loop)

Each solver cites the reference lines it follows; the same torch ops are used in
the same order, so on one machine the results are bit-identical to the
reference's (pinned by tests/golden/throughput_tiny.npz, produced by the
reference itself).  One position id serves the whole batch, and the rotary
embedding is the half-split form (the reference does not permute weights for
this instruction set).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from oracle.pyvm import rms_norm
from thor_megakernels_b200.demos.throughput.instructions import (
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
from thor_megakernels_b200.llama import apply_rotary_pos_emb


def _block(size: int, idx: int) -> tuple[int, int]:
    return size * idx, size * (idx + 1)


def _matmul(a, b):
    # einsum(matA, matB, "a i, b i -> a b") of the reference (:26-31)
    return torch.einsum("ai,bi->ab", a, b)


def pre_attn_layer_norm(g: Globals, ins: PreAttnLayerNorm):
    """:44-70"""
    b = ins.batch_start_idx
    bb = b // g.matmul_batch_block_size
    if ins.layer_idx > 0:
        assert g.barriers[ins.layer_idx - 1, ins.prev_opcode() - 1, bb, 0] == g.num_output_blocks()
    g.rms_rope_intermediates[b] = rms_norm(g.hidden_states[b], g.attn_ln_weights[ins.layer_idx], g.rms_norm_eps)
    g.barriers[ins.layer_idx, ins.opcode() - 1, bb, 0] += 1


def qkv_matmul_rope_append(g: Globals, ins: QKV_MatMulRopeAppend):
    """:73-170: matmul of a 128 x 128 block, half-split rotary embedding on Q and K
    blocks (computed in fp32 against the fp32 tables, stored as bf16), K / V blocks
    written to the cache at pos_id for all 128 sequences."""
    r0, r1 = _block(g.matmul_batch_block_size, ins.batch_start_idx)
    c0, c1 = _block(g.matmul_output_block_size, ins.qkv_block_idx)
    pos, d = g.pos_id, g.head_dim
    assert g.barriers[ins.layer_idx, ins.prev_opcode() - 1, ins.batch_start_idx, 0] == g.matmul_batch_block_size
    out = torch.einsum("oi,bi->bo", g.qkv_proj_weights[ins.layer_idx, c0:c1], g.rms_rope_intermediates[r0:r1])
    k_start = g.num_attention_heads * d
    v_start = k_start + g.num_kv_heads * d
    mode = "q" if c0 < k_start else ("k" if c0 < v_start else "v")
    if mode in "qk":
        arr = out.view(*out.shape[:-1], -1, d)
        roped, _ = apply_rotary_pos_emb(q=arr, k=arr, cos=g.rope_cos[pos], sin=g.rope_sin[pos], unsqueeze_dim=-2)
        out = roped.reshape(*out.shape)
    heads_here = g.matmul_output_block_size // d
    if mode == "q":
        g.post_ln_rope_q[r0:r1, c0:c1] = out
    else:
        arr = out.view(*out.shape[:-1], -1, d)
        first = (c0 - (k_start if mode == "k" else v_start)) // d
        cache = g.k_cache if mode == "k" else g.v_cache
        cache[ins.layer_idx, r0:r1, pos, first : first + heads_here] = arr
    start_bar = c0 // d
    g.barriers[ins.layer_idx, ins.opcode() - 1, ins.batch_start_idx, start_bar : start_bar + heads_here] = 1


def attention_decode(g: Globals, ins: AttentionDecode):
    """:173-217: fp32 scores, softmax and weighted sum over rows 0..pos_id"""
    b, kvh = ins.batch_start_idx, ins.kv_head_idx
    group = g.num_attention_heads // g.num_kv_heads
    seq_len = g.pos_id + 1
    q0, q1 = _block(group, kvh)
    bb = b // g.matmul_batch_block_size
    bars = g.barriers[ins.layer_idx, ins.prev_opcode() - 1, bb]
    assert all(bars[kvh * group + i] == 1 for i in range(group))
    assert bars[g.num_attention_heads + kvh] == 1 and bars[g.num_attention_heads + g.num_kv_heads + kvh] == 1
    q = g.post_ln_rope_q[b].view(-1, g.head_dim)[q0:q1]
    k = g.k_cache[ins.layer_idx, b, :seq_len, kvh]
    v = g.v_cache[ins.layer_idx, b, :seq_len, kvh]
    scores = torch.einsum("hi,ti->ht", q.float(), k.float()) * g.attn_scale
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("ht,to->ho", probs.float(), v.float())
    g.attn_out[b].view(-1, g.head_dim)[q0:q1] = out
    g.barriers[ins.layer_idx, ins.opcode() - 1, bb, 0] += 1


def _matmul_add(g, ins, x, w, expected):
    r0, r1 = _block(g.matmul_batch_block_size, ins.batch_start_idx)
    c0, c1 = _block(g.matmul_output_block_size, ins.output_block_idx)
    assert g.barriers[ins.layer_idx, ins.prev_opcode() - 1, ins.batch_start_idx, 0] == expected
    g.hidden_states[r0:r1, c0:c1] += _matmul(x[r0:r1], w[ins.layer_idx, c0:c1])
    g.barriers[ins.layer_idx, ins.opcode() - 1, ins.batch_start_idx, 0] += 1


def o_proj_residual(g: Globals, ins: O_ProjResidual):
    """:220-252"""
    _matmul_add(g, ins, g.attn_out, g.o_proj_weights, g.matmul_batch_block_size * g.num_kv_heads)


def pre_mlp_layer_norm(g: Globals, ins: PreMLP_Norm):
    """:255-281"""
    b = ins.batch_start_idx
    bb = b // g.matmul_batch_block_size
    assert g.barriers[ins.layer_idx, ins.prev_opcode() - 1, bb, 0] == g.num_output_blocks()
    g.rms_gate_intermediates[b] = rms_norm(g.hidden_states[b], g.mlp_ln_weights[ins.layer_idx], g.rms_norm_eps)
    g.barriers[ins.layer_idx, ins.opcode() - 1, bb, 0] += 1


def gate_silu(g: Globals, ins: GateSilu):
    """:284-320: silu_out block = bf16(silu(bf16 gate matmul))"""
    r0, r1 = _block(g.matmul_batch_block_size, ins.batch_start_idx)
    c0, c1 = _block(g.matmul_output_block_size, ins.output_block_idx)
    assert g.barriers[ins.layer_idx, ins.prev_opcode() - 1, ins.batch_start_idx, 0] == g.matmul_batch_block_size
    g.silu_out[r0:r1, c0:c1] = F.silu(_matmul(g.rms_gate_intermediates[r0:r1], g.gate_proj_weights[ins.layer_idx, c0:c1]))
    g.barriers[ins.layer_idx, ins.opcode() - 1, ins.batch_start_idx, ins.output_block_idx] += 1


def up_matmul(g: Globals, ins: UpMatMul):
    """:323-365: silu_out block *= bf16 up matmul"""
    r0, r1 = _block(g.matmul_batch_block_size, ins.batch_start_idx)
    c0, c1 = _block(g.matmul_output_block_size, ins.output_block_idx)
    assert g.barriers[ins.layer_idx, ins.prev_opcode() - 1, ins.batch_start_idx, ins.output_block_idx] == 1
    up = _matmul(g.rms_gate_intermediates[r0:r1], g.up_proj_weights[ins.layer_idx, c0:c1])
    g.silu_out[r0:r1, c0:c1] = up * g.silu_out[r0:r1, c0:c1]
    g.barriers[ins.layer_idx, ins.opcode() - 1, ins.batch_start_idx, 0] += 1


def down_proj_residual(g: Globals, ins: DownProjResidual):
    """:368-402"""
    _matmul_add(g, ins, g.silu_out, g.down_proj_weights, g.num_intermediate_blocks())


def pre_lm_head_rms(g: Globals, ins: PreLMHeadRMS):
    """:405-434"""
    b = ins.batch_start_idx
    bb = b // g.matmul_batch_block_size
    last = g.num_hidden_layers - 1
    assert g.barriers[last, ins.prev_opcode() - 1, bb, 0] == g.num_output_blocks()
    g.rms_lm_head_intermediates[b] = rms_norm(g.hidden_states[b], g.lm_head_norm_weights, g.rms_norm_eps)
    g.barriers[last, ins.opcode() - 1, bb, 0] += 1


def lm_head(g: Globals, ins: LM_Head):
    """:437-465"""
    r0, r1 = _block(g.matmul_batch_block_size, ins.batch_start_idx)
    c0, c1 = _block(g.matmul_output_block_size, ins.output_block_idx)
    assert g.barriers[g.num_hidden_layers - 1, ins.prev_opcode() - 1, ins.batch_start_idx, 0] == g.matmul_batch_block_size
    g.logits[r0:r1, c0:c1] = _matmul(g.rms_lm_head_intermediates[r0:r1], g.lm_head_weights[c0:c1])


INSTRUCTION_TO_SOLVER = {
    PreAttnLayerNorm: pre_attn_layer_norm, QKV_MatMulRopeAppend: qkv_matmul_rope_append, AttentionDecode: attention_decode,
    O_ProjResidual: o_proj_residual, PreMLP_Norm: pre_mlp_layer_norm, GateSilu: gate_silu, UpMatMul: up_matmul,
    DownProjResidual: down_proj_residual, PreLMHeadRMS: pre_lm_head_rms, LM_Head: lm_head,
}


def interpret_with_pyvm(g: Globals, instructions, instruction_to_solver=INSTRUCTION_TO_SOLVER):
    for ins in instructions:
        instruction_to_solver[type(ins)](g, ins)
