"""Batched ("throughput") instruction set: ten opcodes for a decode step over
``batch_size`` sequences, matmuls cut into 128-sequence x 128-output blocks.

Wire format (opcode, then the dataclass fields in order) and counter protocol
follow the reference's ``megakernels/demos/throughput/instructions.py:9-223``.
Instructions carry a ``pool`` tag (``memory`` for the norms and attention,
``compute`` for the matmuls) that the ``pool`` assignment policy uses.
"""
from __future__ import annotations

from dataclasses import dataclass

from torch import Tensor

from ...instructions import BaseGlobals, Instruction
from ...utils import assert_div


@dataclass
class Globals(BaseGlobals):
    # activation buffers, one row per sequence
    rms_rope_intermediates: Tensor
    rms_gate_intermediates: Tensor
    rms_lm_head_intermediates: Tensor
    post_ln_rope_q: Tensor
    attn_out: Tensor
    silu_out: Tensor
    logits: Tensor

    batch_size: int
    matmul_batch_block_size: int
    matmul_output_block_size: int
    norm_block_size: int

    def qkv_dim(self) -> int:
        return (self.num_attention_heads + 2 * self.num_kv_heads) * self.head_dim

    def num_batch_blocks(self) -> int:
        return assert_div(self.batch_size, self.matmul_batch_block_size)

    def num_output_blocks(self) -> int:
        return assert_div(self.hidden_size, self.matmul_output_block_size)

    def num_intermediate_blocks(self) -> int:
        return assert_div(self.intermediate_size, self.matmul_output_block_size)

    def num_vocab_blocks(self) -> int:
        return assert_div(self.vocab_size, self.matmul_output_block_size)


class ComputeInstruction(Instruction):
    @classmethod
    def tags(cls):
        return {"pool": "compute"}


class MemoryInstruction(Instruction):
    @classmethod
    def tags(cls):
        return {"pool": "memory"}


def _op(code: int, prev):
    """Class decorator: opcode and the opcode whose counters the instruction waits on."""
    def wrap(cls):
        cls.opcode = classmethod(lambda c: code)
        cls.prev_opcode = classmethod(lambda c: prev() if callable(prev) else prev)
        return cls
    return wrap


@_op(1, lambda: 8)
@dataclass
class PreAttnLayerNorm(MemoryInstruction):
    """RMSNorm of one sequence's residual stream before attention."""
    layer_idx: int
    batch_start_idx: int


@_op(2, 1)
@dataclass
class QKV_MatMulRopeAppend(ComputeInstruction):
    """128 sequences x 128 QKV outputs: matmul, rotary embedding on Q and K
    (half-split form), K and V appended to the cache."""
    layer_idx: int
    batch_start_idx: int
    qkv_block_idx: int


@_op(3, 2)
@dataclass
class AttentionDecode(MemoryInstruction):
    layer_idx: int
    batch_start_idx: int
    kv_head_idx: int


@dataclass
class MatMulAdd(ComputeInstruction):
    layer_idx: int
    batch_start_idx: int
    output_block_idx: int


@_op(4, 3)
@dataclass
class O_ProjResidual(MatMulAdd):
    pass


@_op(5, 4)
@dataclass
class PreMLP_Norm(MemoryInstruction):
    layer_idx: int
    batch_start_idx: int


@_op(6, 5)
@dataclass
class GateSilu(ComputeInstruction):
    """gate matmul + SiLU"""
    layer_idx: int
    batch_start_idx: int
    output_block_idx: int


@_op(7, 6)
@dataclass
class UpMatMul(ComputeInstruction):
    """up matmul times the stored SiLU(gate)"""
    layer_idx: int
    batch_start_idx: int
    output_block_idx: int


@_op(8, 7)
@dataclass
class DownProjResidual(MatMulAdd):
    pass


@_op(9, 8)
@dataclass
class PreLMHeadRMS(MemoryInstruction):
    layer_idx: int  # unused (always 0); kept for the wire format
    batch_start_idx: int


@_op(10, 9)
@dataclass
class LM_Head(ComputeInstruction):
    batch_start_idx: int
    output_block_idx: int
