"""Small host helpers shared by the schedule builders and the model container.

Mirrors the helper surface of the reference's ``megakernels/utils.py``:
``assert_div`` (:17-19), ``compute_shard_bounds`` (:22-36),
``load_safetensors_repo`` (:39-97), ``trepr`` (:100-104), ``get_sm_count``
(:107-109).
"""
from __future__ import annotations

import json
import os
from pathlib import Path

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


def compute_shard_bounds(tensor_shape, dim: int, num_shards: int, shard_index: int) -> slice:
    """Range of ``dim`` that shard ``shard_index`` of ``num_shards`` holds; the
    first ``size % num_shards`` shards are one element longer (reference
    utils.py:22-36)."""
    size = tensor_shape[dim]
    base, extra = divmod(size, num_shards)
    start = shard_index * base + min(shard_index, extra)
    return slice(start, start + base + (1 if shard_index < extra else 0))


def load_safetensors_repo(repo_path, include_parameters: set[str], device, tp_rank: int = 0, tp_size: int = 1,
                          tp_map: dict[str, int] | None = None) -> dict[str, Tensor]:
    """Tensors named in ``include_parameters`` from a checkpoint directory that
    holds either ``model.safetensors`` or ``model.safetensors.index.json`` plus
    its shard files.  With ``tp_size > 1`` a parameter listed in ``tp_map`` is
    read only in part: its ``tp_rank``-th slice along the mapped dimension (0 or
    1), so a rank never materialises the other ranks' weights (reference
    utils.py:39-97)."""
    from safetensors import safe_open

    repo_path = Path(repo_path)
    tp_map = tp_map or {}
    single = repo_path / "model.safetensors"
    if single.exists():
        files = [single]
    else:
        index_file = repo_path / "model.safetensors.index.json"
        if not index_file.exists():
            raise FileNotFoundError(f"Could not find model.safetensors or model.safetensors.index.json in {repo_path}")
        weight_map = json.loads(index_file.read_text())["weight_map"]
        files = sorted({repo_path / fname for name, fname in weight_map.items() if name in include_parameters})

    out: dict[str, Tensor] = {}
    for file in files:
        with safe_open(str(file), framework="pt", device=str(device)) as f:
            for name in f.keys():
                if name not in include_parameters:
                    continue
                dim = tp_map.get(name) if tp_size > 1 else None
                if dim is None:
                    out[name] = f.get_tensor(name)
                    continue
                if dim not in (0, 1):
                    raise ValueError(f"Unsupported split dimension: {dim}")
                part = f.get_slice(name)
                bounds = compute_shard_bounds(part.get_shape(), dim, tp_size, tp_rank)
                out[name] = part[bounds] if dim == 0 else part[:, bounds]
    return out


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
