"""TEST INFRASTRUCTURE ONLY - PyTorch (CPU) interpreter of the latency
instruction set, restating the reference's oracle

    megakernels/python_vm.py:83-95                      (interpreter loop)
    megakernels/demos/latency/python_vm.py:23-404       (per-opcode solvers)

Each solver cites the reference lines it follows.  The same torch ops are used
in the same order, so on one machine the results are bit-identical to the
reference's; ``tests/golden/`` pins that with vectors produced by the reference
itself.  The hard-coded 1B constants of the reference's barrier asserts
(``== 512``, ``== 128``; latency/python_vm.py:110,132,176,255) are written as
the shape expressions they stand for.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor

from thor_megakernels_b200.demos.latency.instructions import (
    AttentionReduction,
    DownProjResidual,
    Globals,
    LayerNorm_QKV_MatVecRopeAppend,
    LayerNormDoubleMatVecSiLU,
    O_ProjResidual,
    PartialAttention,
    RMS_LM_Head,
)
from thor_megakernels_b200.instructions import NoOp
from thor_megakernels_b200.llama import apply_rotary_pos_emb_interleaved


def _rows(block_size: int, block_idx: int) -> tuple[int, int]:
    return block_size * block_idx, block_size * (block_idx + 1)


def _mv(mat: Tensor, vec: Tensor) -> Tensor:
    # einsum(mat, vec, "o i, i -> o") of the reference (latency/python_vm.py:47)
    return torch.einsum("oi,i->o", mat, vec)


def rms_norm(inp: Tensor, weight: Tensor, eps: float) -> Tensor:
    """latency/python_vm.py:50-56: fp32 statistics, round to the input dtype,
    then scale by the weight in that dtype."""
    x = inp.to(torch.float32)
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return weight * x.to(inp.dtype)


def matvec_with_residual(mat, vec, residual, block_size, start_block, end_block, reduction_size, reduction_idx):
    """latency/python_vm.py:59-80: per 16-row block, one 2048-column slice,
    bf16 result added in place to the bf16 residual."""
    c0, c1 = _rows(reduction_size, reduction_idx)
    for b in range(start_block, end_block):
        r0, r1 = _rows(block_size, b)
        residual[r0:r1] += _mv(mat[r0:r1, c0:c1], vec[c0:c1]).to(residual.dtype)


def o_proj_residual(g: Globals, ins: O_ProjResidual):
    """latency/python_vm.py:83-104."""
    assert g.barriers[ins.layer_idx, ins.prev_opcode() - 1, 0] == g.num_attention_heads
    assert ins.start_block_idx == ins.end_block_idx - 1 and ins.reduction_block_idx == 0
    # the reference passes matvec_reduction_size (2048), which is the whole input
    # width for the only model it supports; wider models reduce over all of it
    matvec_with_residual(g.o_proj_weights[ins.layer_idx], g.attn_out, g.hidden_states, g.o_proj_block_size,
                         ins.start_block_idx, ins.end_block_idx, g.num_attention_heads * g.head_dim,
                         ins.reduction_block_idx)
    g.barriers[ins.layer_idx, ins.opcode() - 1, 0] += ins.end_block_idx - ins.start_block_idx


def down_proj_residual(g: Globals, ins: DownProjResidual):
    """latency/python_vm.py:107-124 (512 = intermediate_size / 16)."""
    assert g.barriers[ins.layer_idx, ins.prev_opcode() - 1, 0] == g.intermediate_size // g.up_gate_proj_block_size
    matvec_with_residual(g.down_proj_weights[ins.layer_idx], g.silu_out, g.hidden_states, g.down_proj_block_size,
                         ins.start_block_idx, ins.end_block_idx, g.matvec_reduction_size, ins.reduction_block_idx)
    g.barriers[ins.layer_idx, ins.opcode() - 1, 0] += ins.end_block_idx - ins.start_block_idx


def layer_norm_double_matvec_silu(g: Globals, ins: LayerNormDoubleMatVecSiLU):
    """latency/python_vm.py:127-165 (128 = hidden_size / 16)."""
    assert g.barriers[ins.layer_idx, ins.prev_opcode() - 1, 0] == g.hidden_size // g.o_proj_block_size
    x = rms_norm(g.hidden_states, g.mlp_ln_weights[ins.layer_idx], g.rms_norm_eps)
    for b in ins.block_idxs:
        r0, r1 = _rows(g.up_gate_proj_block_size, b)
        up = _mv(g.up_proj_weights[ins.layer_idx][r0:r1], x)
        gate = _mv(g.gate_proj_weights[ins.layer_idx][r0:r1], x)
        g.silu_out[r0:r1] = F.silu(gate) * up
        g.barriers[ins.layer_idx, ins.opcode() - 1, 0] += 1


def layer_norm_matvec_rope_append(g: Globals, ins: LayerNorm_QKV_MatVecRopeAppend):
    """latency/python_vm.py:168-248 (512 = down-projection blocks x column slices)."""
    layer = ins.layer_idx
    if layer > 0:
        expected = (g.hidden_size // g.down_proj_block_size) * (g.intermediate_size // g.matvec_reduction_size)
        assert g.barriers[layer - 1, ins.prev_opcode() - 1, 0] == expected
    x = rms_norm(g.hidden_states, g.attn_ln_weights[layer], g.rms_norm_eps)
    pos = g.pos_id
    k_start = g.num_attention_heads * g.head_dim
    v_start = k_start + g.num_kv_heads * g.head_dim
    blocks_per_head = g.head_dim // g.qkv_block_size
    for b in range(ins.start_output_block_idx, ins.end_output_block_idx):
        r0, r1 = _rows(g.qkv_block_size, b)
        out = _mv(g.qkv_proj_weights[layer][r0:r1], x)
        if r0 < v_start:  # Q and K rows get the rotary embedding
            head = torch.zeros(1, g.head_dim, device=out.device, dtype=out.dtype)
            h0 = r0 % g.head_dim
            head[:, h0 : h0 + (r1 - r0)] = out
            roped, _ = apply_rotary_pos_emb_interleaved(q=head, k=head, cos=g.rope_cos[pos], sin=g.rope_sin[pos],
                                                        unsqueeze_dim=0)
            out = roped[:, h0 : h0 + (r1 - r0)].view(-1)
        if r0 < k_start:
            g.post_ln_rope_q[r0:r1] = out
        elif r0 < v_start:
            g.k_cache[layer, :, pos].view(-1)[r0 - k_start : r1 - k_start] = out
        else:
            g.v_cache[layer, :, pos].view(-1)[r0 - v_start : r1 - v_start] = out
        # the reference writes `block_idx // 4`, i.e. blocks per head at head_dim 64
        g.barriers[layer, ins.opcode() - 1, b // blocks_per_head] += 1


def rms_lm_head(g: Globals, ins: RMS_LM_Head):
    """latency/python_vm.py:251-274."""
    expected = (g.hidden_size // g.down_proj_block_size) * (g.intermediate_size // g.matvec_reduction_size)
    assert g.barriers[g.num_hidden_layers - 1, ins.prev_opcode() - 1, 0] == expected
    x = rms_norm(g.hidden_states, g.lm_head_norm_weights, g.rms_norm_eps)
    for b in range(ins.start_output_block_idx, ins.end_output_block_idx):
        r0, r1 = _rows(g.lm_head_block_size, b)
        g.logits[r0:r1] = _mv(g.lm_head_weights[r0:r1], x)


def partial_attention(g: Globals, ins: PartialAttention):
    """latency/python_vm.py:277-346: fp32 scores, softmax and weighted sum over
    this slice of the cache; lse is log2 of the natural-exponent sum."""
    group = g.num_attention_heads // g.num_kv_heads
    blocks_per_head = g.head_dim // g.qkv_block_size
    ready = g.barriers[ins.layer_idx, ins.prev_opcode() - 1]
    for i in range(group):
        assert ready[ins.kv_head_idx * group + i] == blocks_per_head
    assert ready[g.num_attention_heads + ins.kv_head_idx] == blocks_per_head
    assert ready[g.num_attention_heads + g.num_kv_heads + ins.kv_head_idx] == blocks_per_head

    seq_len = g.pos_id + 1
    total_blocks = math.ceil(seq_len / g.attn_kv_block_size)
    per_partial = math.ceil(total_blocks / ins.num_partials)
    b0 = ins.partial_idx * per_partial
    b1 = min(b0 + per_partial, total_blocks)
    t0 = b0 * g.attn_kv_block_size
    t1 = min(b1 * g.attn_kv_block_size, seq_len)

    k = g.k_cache[ins.layer_idx, 0, t0:t1, ins.kv_head_idx]
    v = g.v_cache[ins.layer_idx, 0, t0:t1, ins.kv_head_idx]
    h0, h1 = ins.kv_head_idx * group, (ins.kv_head_idx + 1) * group
    q = g.post_ln_rope_q.view(g.num_attention_heads, -1)[h0:h1]

    scores = torch.einsum("hi,ki->hk", q.float(), k.float()) * g.attn_scale
    probs = torch.softmax(scores, dim=-1)
    lse = torch.log2(torch.sum(torch.exp(scores), dim=-1))
    out = torch.einsum("hk,ko->ho", probs.float(), v.float())

    if g.skip_attn_reduction:
        g.attn_out.view(g.num_attention_heads, -1)[h0:h1, :] = out
        g.barriers[ins.layer_idx, AttentionReduction.opcode() - 1, 0] += h1 - h0
    else:
        g.attn_lse_intermediates[h0:h1, ins.partial_idx] = lse
        g.attn_out_intermediates[h0:h1, ins.partial_idx] = out
        g.barriers[ins.layer_idx, ins.opcode() - 1, h0:h1] += 1


def attention_reduction(g: Globals, ins: AttentionReduction):
    """latency/python_vm.py:349-393: weights exp2(lse - max)."""
    h0 = ins.head_start_idx
    h1 = h0 + g.attn_reduction_size
    assert g.barriers[ins.layer_idx, ins.prev_opcode() - 1, h0] == ins.num_partials
    picks = torch.tensor(ins.reduction_list, dtype=torch.long, device=g.hidden_states.device)
    lses = g.attn_lse_intermediates[h0:h1, picks]
    outs = g.attn_out_intermediates[h0:h1, picks]
    weights = (lses - torch.max(lses, dim=-1, keepdim=True).values).exp2()
    denom = weights.sum(dim=-1, keepdim=True)
    merged = (outs * weights.unsqueeze(-1)).sum(dim=1) / denom
    if ins.is_terminal:
        g.attn_out.view(g.num_attention_heads, -1)[h0:h1] = merged
    else:
        g.attn_lse_intermediates[h0:h1, ins.output_partial_idx] = denom.log()
        g.attn_out_intermediates[h0:h1, ins.output_partial_idx] = merged
    g.barriers[ins.layer_idx, ins.opcode() - 1, 0] += g.attn_reduction_size


def _noop(g, ins):
    return None


INSTRUCTION_TO_SOLVER = {
    NoOp: _noop,
    O_ProjResidual: o_proj_residual,
    DownProjResidual: down_proj_residual,
    LayerNormDoubleMatVecSiLU: layer_norm_double_matvec_silu,
    LayerNorm_QKV_MatVecRopeAppend: layer_norm_matvec_rope_append,
    RMS_LM_Head: rms_lm_head,
    PartialAttention: partial_attention,
    AttentionReduction: attention_reduction,
}


def interpret_with_pyvm(g: Globals, instructions, instruction_to_solver=INSTRUCTION_TO_SOLVER):
    """python_vm.py:83-87: run the instructions in the given (topological) order."""
    for ins in instructions:
        instruction_to_solver[type(ins)](g, ins)


class PyVM_Interpreter:
    """python_vm.py:90-95."""

    def __init__(self, instruction_to_solver=INSTRUCTION_TO_SOLVER):
        self.instruction_to_solver = instruction_to_solver

    def interpret(self, g: Globals, instructions):
        interpret_with_pyvm(g, instructions, self.instruction_to_solver)


def pyvm_step(model, schedule, instructions, input_ids: Tensor, pos_id: int):
    """One decode step the way the reference's PyVM_Generator.run does it
    (generators.py:179-201): embed, zero the counters, interpret, then RMSNorm +
    LM head + argmax through the model's own head."""
    from thor_megakernels_b200.model_types import BatchState

    g = schedule.globs
    state = model.model.embed_tokens(BatchState(input_ids=input_ids))
    g.hidden_states[:] = state.hidden_states
    g.barriers.zero_()
    g.pos_id = pos_id
    interpret_with_pyvm(g, instructions)
    state.hidden_states = g.hidden_states
    return model.lm_head(state).output_ids
