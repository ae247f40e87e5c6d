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


def nrmse(got: torch.Tensor, ref: torch.Tensor) -> float:
    g, r = got.detach().float().cpu().flatten(), ref.detach().float().cpu().flatten()
    return float((g - r).norm() / r.norm().clamp_min(1e-12))


def load_sensitivity(name: str):
    """Distance of an exactly rounded restatement from the golden vectors
    (tests/golden/make_sensitivity.py)."""
    return dict(np.load(GOLDEN / f"{name}_sensitivity.npz"))


class exact_matvecs:
    """While active, the oracle's matvecs are computed in float64 and rounded
    once: the result any summation order would give with perfect accumulation."""

    def __enter__(self):
        from oracle import pyvm

        self._pyvm, self._plain = pyvm, pyvm._mv
        pyvm._mv = lambda mat, vec: (mat.double() @ vec.double()).to(mat.dtype)
        return self

    def __exit__(self, *exc):
        self._pyvm._mv = self._plain
        return False


def assert_within_rounding_noise(name: str, got, ref, exact, factor: float = 2.0, floor: float = 2e-3):
    """``got`` (the kernel) may differ from ``ref`` (the reference's result) by
    at most ``factor`` times what ``exact`` (the same computation with exactly
    rounded matvecs) differs from it, measured as NRMSE and as max-abs, plus a
    small floor of one part in 500."""
    e_got, e_exact = nrmse(got, ref), nrmse(exact, ref)
    m_got = float((got.detach().float().cpu() - ref.detach().float().cpu()).abs().max())
    m_exact = float((exact.detach().float().cpu() - ref.detach().float().cpu()).abs().max())
    scale = float(ref.detach().float().abs().max())
    rep = dict(name=name, nrmse=e_got, exact_nrmse=e_exact, max_abs=m_got, exact_max_abs=m_exact)
    assert e_got <= factor * e_exact + floor, rep
    assert m_got <= factor * m_exact + 4 * floor * scale, rep
    return rep


def assert_parity(name: str, got, ref, exact, factor: float = 2.0):
    """The stated tolerance, |got - ref| <= 3e-2 + 1e-2 |ref| on every element;
    where the computation is deep enough that even an exactly rounded
    restatement (``exact``) leaves that band, the kernel must instead stay
    within ``factor`` times that restatement's own distance from ``ref``."""
    rep = mismatch_report(name, got, ref)
    if rep["violations"] == 0:
        return rep
    rep.update(assert_within_rounding_noise(name, got, ref, exact, factor))
    return rep
