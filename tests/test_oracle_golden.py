"""Pins the CPU side to vectors produced by the reference's own code
(tests/golden/, made by tests/golden/make_golden.py):

* the model container (stacked weights, rotary tables) and the four queue
  assignment policies reproduce the reference's tensors bit for bit;
* the oracle interpreter (oracle/pyvm.py) reproduces the reference
  interpreter's buffers for every decode step of the small case.
"""
import hashlib

import numpy as np
import pytest
import torch

from helpers import bf16_from_u16, build_model, build_schedule, load_golden, load_prefill


def sha(t: torch.Tensor) -> str:
    raw = t.detach().contiguous()
    if raw.dtype == torch.bfloat16:
        raw = raw.view(torch.int16)
    return hashlib.sha256(raw.numpy().tobytes()).hexdigest()


@pytest.fixture(scope="module")
def tiny_cpu():
    meta, arrays = load_golden("tiny")
    return meta, arrays, build_model(meta["config"], meta["max_len"], device="cpu")


def same_cpu_kernels(meta) -> bool:
    """bf16 matmuls pick ISA-specific kernels; bitwise equality is only promised
    on the instruction set the vectors were generated with."""
    return torch.backends.cpu.get_cpu_capability() == meta["cpu_capability"] and torch.__version__ == meta["torch"]


def test_model_container_matches_reference(tiny_cpu):
    meta, arrays, model = tiny_cpu
    sp = model.stacked_params
    got = {"qkv_proj": sp.qkv_proj, "o_proj": sp.o_proj, "up_proj": sp.up_proj, "gate_proj": sp.gate_proj,
           "down_proj": sp.down_proj, "lm_head": model.lm_head.lm_head.weight}
    for name, t in got.items():
        assert sha(t) == meta["weights_sha256"][name], name
    assert sha(model.model.rope_cos) == meta["rope_sha256"]["cos"]
    assert sha(model.model.rope_sin) == meta["rope_sha256"]["sin"]


@pytest.mark.parametrize("mode", ["rr", "zz", "wave", "dag"])
def test_queue_tensors_match_reference_tiny(tiny_cpu, mode):
    meta, arrays, model = tiny_cpu
    sched = build_schedule(model, mode)
    assert len(sched.dag_nodes) == meta["dag_nodes"]
    assert list(sched.globs.instructions.shape) == meta["instructions_shape"][mode]
    assert sha(sched.globs.instructions) == meta["instructions_sha256"][mode]
    if mode == "rr":
        assert np.array_equal(sched.globs.instructions.numpy(), arrays["instructions_rr"])


@pytest.mark.parametrize("mode", ["rr", "zz", "wave", "dag"])
def test_queue_tensors_match_reference_llama1b(mode):
    """Llama-3.2-1B shapes on 148 workers, without materialising any weight."""
    from thor_megakernels_b200.demos.latency.scheduler import LatencyScheduleBuilder
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig
    from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    meta, _ = load_golden("llama1b")
    with torch.device("meta"):
        model = LlamaForCausalLM(LlamaConfig(**meta["config"]), ExtraModelConfig(interleave_rope=True, max_len_override=8))
        model.device = torch.device("meta")
        model.stack_params()
        model.setup_caches()
    sched = LatencyScheduleBuilder.build(model)
    sched.globs.device = "cpu"
    tensorize_instructions(sched.globs, assign_to_sms(mode, schedule=sched))
    assert len(sched.dag_nodes) == meta["dag_nodes"] == 9428
    assert list(sched.globs.instructions.shape) == meta["instructions_shape"][mode]
    assert sha(sched.globs.instructions) == meta["instructions_sha256"][mode]


def test_oracle_reproduces_reference_interpreter(tiny_cpu):
    from oracle import pyvm

    meta, arrays, model = tiny_cpu
    assert meta["oracle_bit_identical"] is True  # checked against the live reference when the vectors were made
    sched = build_schedule(model)
    n = load_prefill(model, arrays)
    exact = same_cpu_kernels(meta)
    g = sched.globs
    for step in range(meta["ntok"]):
        pos = n + step
        out = pyvm.pyvm_step(model, sched, sched.get_linear_instructions(), torch.tensor([[int(arrays["tokens"][step])]]), pos)
        want = {
            "hidden_states": bf16_from_u16(arrays["hidden"][step]),
            "post_ln_rope_q": bf16_from_u16(arrays[f"q_step{step}"]),
            "attn_out": bf16_from_u16(arrays[f"attn_out_step{step}"]),
            "silu_out": bf16_from_u16(arrays[f"silu_out_step{step}"]),
            "logits": bf16_from_u16(arrays[f"logits_step{step}"]),
        }
        for name, ref in want.items():
            got = getattr(g, name)
            if exact:
                assert torch.equal(got, ref), (step, name)
            else:
                assert torch.allclose(got.float(), ref.float(), atol=3e-2, rtol=1e-2), (step, name)
        assert np.array_equal(g.barriers.numpy(), arrays[f"barriers_step{step}"])
        k_row = model.stacked_kv_cache[0][:, 0, pos]
        if exact:
            assert torch.equal(k_row, bf16_from_u16(arrays[f"k_row_step{step}"]))
            assert int(out) == int(arrays["tokens"][step + 1])


def test_prefill_matches_reference(tiny_cpu):
    from thor_megakernels_b200.model_types import BatchState

    meta, arrays, model = tiny_cpu
    prompt = torch.from_numpy(arrays["prompt"]).long()
    n = prompt.shape[1]
    model.stacked_kv_cache[0].zero_()
    model.stacked_kv_cache[1].zero_()
    out = model(BatchState(input_ids=prompt, position_ids=torch.arange(n)[None], seq_len=n))
    k = model.stacked_kv_cache[0][:, 0, :n]
    if same_cpu_kernels(meta):
        assert torch.equal(k, bf16_from_u16(arrays["prefill_k"]))
        assert int(out.output_ids[0, -1]) == int(arrays["tokens"][0])
    else:
        assert torch.allclose(k.float(), bf16_from_u16(arrays["prefill_k"]).float(), atol=3e-2, rtol=1e-2)
