"""Shared test utilities: golden fixtures, seeded models, tolerance checks."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"

# bf16 hidden states and logits: |a - ref| <= 3e-2 + 1e-2 * |ref|
ATOL, RTOL = 3e-2, 1e-2


def load_golden(name: str):
    meta = json.loads((GOLDEN / f"{name}.json").read_text())
    arrays = dict(np.load(GOLDEN / f"{name}.npz"))
    return meta, arrays


def bf16_from_u16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.astype(np.int16)).view(torch.bfloat16)


def build_model(meta_or_cfg, max_len: int, device="cpu", seed: int = 0):
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig

    cfg = meta_or_cfg if isinstance(meta_or_cfg, dict) else dict(meta_or_cfg)
    return LlamaForCausalLM.random_init(
        LlamaConfig(**cfg), ExtraModelConfig(interleave_rope=True, max_len_override=max_len), seed=seed, device=device
    )


def build_schedule(model, mode: str = "rr", **kwargs):
    from thor_megakernels_b200.demos.latency.scheduler import LatencyScheduleBuilder
    from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    sched = LatencyScheduleBuilder.build(model, **kwargs)
    tensorize_instructions(sched.globs, assign_to_sms(mode, schedule=sched))
    return sched


def load_prefill(model, arrays):
    """Put the golden prefill K/V rows into the model's cache."""
    k = bf16_from_u16(arrays["prefill_k"]).to(model.device)
    v = bf16_from_u16(arrays["prefill_v"]).to(model.device)
    n = k.shape[1]
    model.stacked_kv_cache[0][:, 0, :n] = k
    model.stacked_kv_cache[1][:, 0, :n] = v
    return n


def mismatch_report(name: str, got: torch.Tensor, ref: torch.Tensor, atol=ATOL, rtol=RTOL):
    g, r = got.detach().float().cpu().flatten(), ref.detach().float().cpu().flatten()
    err = (g - r).abs()
    bad = err > (atol + rtol * r.abs())
    return {
        "name": name,
        "max_abs": float(err.max()) if err.numel() else 0.0,
        "exact_fraction": float((g == r).float().mean()) if err.numel() else 1.0,
        "violations": int(bad.sum()),
        "worst_ref": float(r[err.argmax()]) if err.numel() else 0.0,
    }


def assert_close(name: str, got: torch.Tensor, ref: torch.Tensor, atol=ATOL, rtol=RTOL):
    rep = mismatch_report(name, got, ref, atol, rtol)
    assert rep["violations"] == 0, rep
    return rep
