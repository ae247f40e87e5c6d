"""Instruction wire format and the per-model table of buffers and constants.

Same public surface as the reference's ``megakernels/instructions.py``:
``BaseGlobals`` (:10-91), ``diff_tensors`` (:94-102), ``Instruction.serialize``
(:105-141) and ``NoOp`` (:144-148).  An instruction serialises to at most 32
int32 words: word 0 is the opcode, then every dataclass field in declaration
order; a list or tuple is written as its length followed by its items and
``None`` as 0.  Opcode 0 (all-zero row) is the padding no-op.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any

from torch import Tensor

from .model_types import DeviceType
from .utils import get_sm_count


@dataclass
class BaseGlobals:
    # stacked weights, layer-major
    qkv_proj_weights: Tensor
    attn_ln_weights: Tensor
    o_proj_weights: Tensor
    mlp_ln_weights: Tensor
    up_proj_weights: Tensor
    gate_proj_weights: Tensor
    down_proj_weights: Tensor
    lm_head_norm_weights: Tensor
    lm_head_weights: Tensor
    k_cache: Tensor
    v_cache: Tensor

    # rotary tables, shared by all layers
    rope_cos: Tensor
    rope_sin: Tensor

    # shape constants
    num_hidden_layers: int
    num_attention_heads: int
    num_kv_heads: int
    head_dim: int
    hidden_size: int
    intermediate_size: int
    vocab_size: int

    attn_scale: float
    rms_norm_eps: float
    device: DeviceType

    hidden_states: Tensor
    barriers: Tensor

    pos_id: int

    def __post_init__(self):
        # Filled by scheduler.tensorize_instructions.
        self.instructions: Tensor | None = None
        self.timings: Tensor | None = None

    # -- worker budget ---------------------------------------------------
    def physical_sm_count(self) -> int:
        return get_sm_count(self.device)

    def sm_count(self) -> int:
        """Number of worker queues: all SMs unless ``set_active_workers`` narrowed it."""
        physical = self.physical_sm_count()
        active = getattr(self, "active_workers", None)
        if active is None:
            return physical
        valid = isinstance(active, int) and not isinstance(active, bool)
        if not valid or active < 1 or active > physical:
            raise ValueError("active_workers must be an integer in 1..physical SM count")
        return active

    def set_active_workers(self, count: int):
        """Restrict the schedule to ``count`` workers.  Queue tensors built for
        another count are dropped (reference instructions.py:63-74)."""
        if type(count) is not int:
            raise ValueError("active worker count must be an integer")
        before = getattr(self, "active_workers", None)
        self.active_workers = count
        try:
            self.sm_count()
        except ValueError:
            self.active_workers = before
            raise
        self.instructions = None
        self.timings = None

    # -- debugging -------------------------------------------------------
    def diff(self, other: "BaseGlobals", skip_kv_cache: bool = False):
        """Print max-abs / mean-relative differences of every activation buffer."""
        for f in dataclasses.fields(self):
            mine = getattr(self, f.name)
            if not isinstance(mine, Tensor):
                continue
            if "weights" in f.name or f.name in ("rope_cos", "rope_sin"):
                continue
            if skip_kv_cache and "cache" in f.name:
                continue
            diff_tensors(mine, getattr(other, f.name), f.name)

    def num_total_heads(self) -> int:
        return self.num_attention_heads + 2 * self.num_kv_heads


def diff_tensors(a: Tensor, b: Tensor, name: str):
    a32, b32 = a.float(), b.float()
    diff = a32 - b32
    adiff = diff.abs()
    rdiff = 2 * adiff / (a32.abs() + b32.abs() + 1e-6)
    print(f"{name}: max adiff: {adiff.max()}, mean rdiff: {rdiff.mean()}")
    return diff, adiff, rdiff


@dataclass
class Instruction:
    @classmethod
    def opcode(cls) -> int:
        raise NotImplementedError

    @classmethod
    def prev_opcode(cls) -> int:
        raise NotImplementedError

    @classmethod
    def tags(cls) -> dict[str, Any]:
        return {}

    def serialize(self) -> list[int]:
        words = [self.opcode()]
        for f in dataclasses.fields(self):
            if f.name == "global_idx":
                continue
            value = getattr(self, f.name)
            if value is None:
                words.append(0)
            elif isinstance(value, int):  # bool is an int: True -> 1
                words.append(value)
            elif isinstance(value, (list, tuple)):
                words.append(len(value))
                words.extend(value)
            else:
                raise ValueError(f"Unsupported field type: {value}")
        return words


@dataclass
class NoOp(Instruction):
    @classmethod
    def opcode(cls) -> int:
        return 0
