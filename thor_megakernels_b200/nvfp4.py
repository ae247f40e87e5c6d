"""Host side of the NVFP4 weight-only path: quantise bf16 weights on the
device and run the fused dequantise-GEMV, both through the C-ABI library.

Storage follows the reference harness's ``Primitive.storage`` / ``quantize`` /
``simt`` (tools/analysis/nvfp4/bench.py:58-84): ``packed`` uint8 ``[rows, k/2]``,
``scales`` uint8 ``[rows, k/16]`` (E4M3 bits), ``tensor_scale`` =
``max(amax / (6*448), 1e-12)``.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from . import _lib


@dataclass
class Nvfp4Weight:
    packed: torch.Tensor        # uint8 [rows, k/2]
    scales: torch.Tensor        # uint8 [rows, k/16]
    tensor_scale: float
    rows: int
    k: int
    decoded: torch.Tensor | None = None  # fp32 [rows, k], only when asked for

    @property
    def nbytes(self) -> int:
        return self.packed.numel() + self.scales.numel()


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def tensor_scale_for(weight: torch.Tensor) -> float:
    return float(np.float32(max(weight.abs().max().item() / (6 * 448), 1e-12)))


def quantize_weight(weight: torch.Tensor, tensor_scale: float | None = None, reference: bool = False) -> Nvfp4Weight:
    """Quantise a contiguous bf16 ``[rows, k]`` CUDA tensor (``k % 16 == 0``)."""
    if weight.device.type != "cuda" or weight.dtype != torch.bfloat16 or not weight.is_contiguous() or weight.ndim != 2:
        raise ValueError("Source must be contiguous device BF16 [rows, k]")
    rows, k = weight.shape
    if k % 16:
        raise ValueError("k must be a multiple of 16")
    ts = tensor_scale_for(weight) if tensor_scale is None else float(tensor_scale)
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=weight.device)
    scales = torch.empty((rows, k // 16), dtype=torch.uint8, device=weight.device)
    decoded = torch.empty((rows, k), dtype=torch.float32, device=weight.device) if reference else None
    lib = _lib.load()
    with torch.cuda.device(weight.device):
        _lib.check(lib.mk_nvfp4_quantize(weight.data_ptr(), packed.data_ptr(), scales.data_ptr(),
                                         decoded.data_ptr() if reference else None, rows, k, ts, _stream(weight)))
    return Nvfp4Weight(packed, scales, ts, rows, k, decoded)


_workspaces: dict = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Split-K scratch for ``gemv`` calls that do not bring their own: one
    buffer per (device, stream), grown on demand.  Calls on one stream run in
    order, so they can share it; calls on different streams get different
    buffers."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)  # zeroed once; calls leave it zeroed
        _workspaces[key] = buf
    return buf


def gemv(weight: Nvfp4Weight | torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None,
         workspace: torch.Tensor | None = None) -> torch.Tensor:
    """``y[b] = W @ x[b]`` for ``x`` of shape ``[k]`` or ``[batch <= 8, k]`` (bf16),
    fp32 accumulation, bf16 result.  ``weight`` is an ``Nvfp4Weight`` (fused
    dequantisation) or a plain bf16 matrix.  ``workspace``: a uint8 CUDA tensor
    of at least ``mk_gemv_workspace_bytes(rows, k)`` bytes for the split-K sums
    (needed when k > 2048); by default a per-stream buffer owned by this module.
    The library call itself never allocates."""
    if x.device.type != "cuda" or x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("x must be a contiguous bf16 CUDA tensor")
    squeeze = x.ndim == 1
    xb = x.view(1, -1) if squeeze else x
    batch, k = xb.shape
    is_packed = isinstance(weight, Nvfp4Weight)
    rows = weight.rows if is_packed else weight.shape[0]
    wk = weight.k if is_packed else weight.shape[1]
    if wk != k:
        raise ValueError(f"x has {k} columns, weight has {wk}")
    y = out if out is not None else torch.empty((batch, rows), dtype=torch.bfloat16, device=x.device)
    lib = _lib.load()
    need = int(lib.mk_gemv_workspace_bytes(rows, k))
    if need and workspace is None:
        workspace = _workspace(x.device, need)
    ws_ptr, ws_bytes = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if need else (None, 0)
    with torch.cuda.device(x.device):
        if is_packed:
            code = lib.mk_gemv(None, weight.packed.data_ptr(), weight.scales.data_ptr(), xb.data_ptr(), y.data_ptr(),
                               rows, k, weight.tensor_scale, 1, batch, ws_ptr, ws_bytes, _stream(x))
        else:
            if weight.dtype != torch.bfloat16 or not weight.is_contiguous():
                raise ValueError("weight must be contiguous bf16")
            code = lib.mk_gemv(weight.data_ptr(), None, None, xb.data_ptr(), y.data_ptr(), rows, k, 1.0, 0, batch,
                               ws_ptr, ws_bytes, _stream(x))
    if code != 0:
        raise _lib.MegakernelError(code, lib.mk_last_error().decode() or f"mk_gemv refused m={rows} k={k} batch={batch}")
    return y.view(-1) if squeeze and out is None else y


def quantize_model(model) -> dict:
    """Quantise every linear of a finalised model container for the NVFP4
    weight-only megakernel: per layer qkv, o, up, gate, down and the LM head.
    up and gate share the tensor scale of their concatenation, as in the
    reference's plan where they are one matrix
    (experimental/native_fp4_vm/model.cu:112-126)."""
    sp = model.stacked_params
    out = {k: [] for k in ("qkv", "o", "up", "gate", "down")}
    for i in range(model.config.num_hidden_layers):
        ug = float(np.float32(max(max(sp.up_proj[i].abs().max().item(), sp.gate_proj[i].abs().max().item()) / (6 * 448), 1e-12)))
        out["qkv"].append(quantize_weight(sp.qkv_proj[i].contiguous()))
        out["o"].append(quantize_weight(sp.o_proj[i].contiguous()))
        out["up"].append(quantize_weight(sp.up_proj[i].contiguous(), ug))
        out["gate"].append(quantize_weight(sp.gate_proj[i].contiguous(), ug))
        out["down"].append(quantize_weight(sp.down_proj[i].contiguous()))
    out["lm_head"] = quantize_weight(model.lm_head.lm_head.weight.data.contiguous())
    return out
