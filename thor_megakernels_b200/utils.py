"""Small host helpers shared by the schedule builders and the model container.

Mirrors the helper surface of the reference's ``megakernels/utils.py``
(``assert_div`` at :17-19, ``get_sm_count`` at :107-109, ``trepr`` at :100-104).
The checkpoint loader (``load_safetensors_repo``) is not part of the decode
hot path and is not provided.
"""
from __future__ import annotations

import os

import torch
from torch import Tensor

# Number of SMs on a B200.  Used when a schedule is built for a device that is
# not visible from this process (CPU-only build and test boxes).
B200_SM_COUNT = 148


def assert_div(a: int, b: int) -> int:
    """Exact integer division; refuses to round (reference utils.py:17-19)."""
    if a % b != 0:
        raise AssertionError(f"{a} is not divisible by {b}")
    return a // b


def get_sm_count(device) -> int:
    """Worker count of ``device`` (reference utils.py:107-109).

    The reference asks CUDA unconditionally.  Schedules here are also built on
    machines without a GPU, so a CPU device reports the B200 count (or the
    value of ``MK_SM_COUNT`` when set) instead of raising.
    """
    override = os.environ.get("MK_SM_COUNT")
    if override:
        return int(override)
    dev = torch.device(device) if not isinstance(device, torch.device) else device
    if dev.type == "cuda" and torch.cuda.is_available():
        return torch.cuda.get_device_properties(dev).multi_processor_count
    return B200_SM_COUNT


def trepr(t: Tensor) -> str:
    """One-line tensor summary used by debug prints (reference utils.py:100-104)."""
    return f"shape={tuple(t.shape)}, sum={t.sum()}, vals={t}"
