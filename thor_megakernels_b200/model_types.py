"""Plain data carriers passed between the decode loop, the model container and
the kernels.  Field names follow the reference's ``megakernels/model_types.py``
(:22-60) so that caller code written against it keeps working; fields that only
the reference's paged-attention serving path used are left out.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor

KV_Cache = tuple[Tensor, Tensor]
DeviceType = torch.device | str


@dataclass
class BatchState:
    """One forward call's inputs and outputs (reference model_types.py:22-41)."""

    input_ids: Tensor
    position_ids: Tensor | None = None
    seq_len: int | None = None
    output_ids: Tensor | None = None
    hidden_states: Tensor | None = None
    position_embeddings: tuple[Tensor, Tensor] | None = None

    def __post_init__(self):
        if self.seq_len is None:
            self.seq_len = self.input_ids.shape[1]


@dataclass
class ExtraModelConfig:
    """Switches that are not part of the Hugging Face config
    (reference model_types.py:44-60)."""

    tp_size: int = 1
    tp_rank: int = 0
    rope_scaling: dict | None = None
    interleave_rope: bool = False
    max_len_override: int | None = None
    max_batch_size: int = 1
