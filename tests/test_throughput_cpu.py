"""Batched ("throughput") instruction set on the CPU: wire format, schedule
builder and the oracle interpreter against golden vectors produced by the
reference itself (tests/golden/make_golden_throughput.py)."""
import hashlib

import numpy as np
import pytest
import torch

from helpers import bf16_from_u16, load_golden


def sha(t):
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def build_tiny(device="cpu"):
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig

    meta, arrays = load_golden("throughput_tiny")
    model = LlamaForCausalLM.random_init(
        LlamaConfig(**meta["config"]),
        ExtraModelConfig(interleave_rope=False, max_len_override=meta["max_len"], max_batch_size=meta["batch"]),
        seed=5, device=device)
    return meta, arrays, model


def load_inputs(sched, model, meta, arrays):
    g = sched.globs
    g.hidden_states[:] = bf16_from_u16(arrays["hidden_in"]).to(g.hidden_states.device)
    g.pos_id = meta["pos_id"]
    g.barriers.zero_()
    model.stacked_kv_cache[0].copy_(bf16_from_u16(arrays["k_in"]))
    model.stacked_kv_cache[1].copy_(bf16_from_u16(arrays["v_in"]))


def test_wire_format_and_counter_chain():
    from thor_megakernels_b200.demos.throughput import instructions as ins

    assert ins.QKV_MatMulRopeAppend(1, 0, 5).serialize()[:4] == [2, 1, 0, 5]
    assert ins.LM_Head(3, 7).serialize()[:3] == [10, 3, 7]
    chain = [ins.PreAttnLayerNorm, ins.QKV_MatMulRopeAppend, ins.AttentionDecode, ins.O_ProjResidual, ins.PreMLP_Norm,
             ins.GateSilu, ins.UpMatMul, ins.DownProjResidual, ins.PreLMHeadRMS, ins.LM_Head]
    assert [c.opcode() for c in chain] == list(range(1, 11))
    assert [c.prev_opcode() for c in chain] == [8, 1, 2, 3, 4, 5, 6, 7, 8, 9]
    assert ins.AttentionDecode.tags()["pool"] == "memory" and ins.UpMatMul.tags()["pool"] == "compute"


def test_queues_match_the_reference_for_every_policy():
    from thor_megakernels_b200.demos.throughput.scheduler import ThroughputScheduleBuilder
    from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    meta, _, model = build_tiny()
    sched = ThroughputScheduleBuilder.build(model)
    assert len(sched.dag_nodes) == meta["dag_nodes"]
    for mode, kw in (("rr", {}), ("zz", {}), ("pool", dict(memory_fraction=0.5))):
        tensorize_instructions(sched.globs, assign_to_sms(mode, schedule=sched, **kw))
        assert sha(sched.globs.instructions) == meta["instructions_sha256"][mode], mode


def test_batch_must_be_a_multiple_of_128():
    from thor_megakernels_b200.demos.throughput.scheduler import ThroughputScheduleBuilder
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig

    meta, _, _ = build_tiny()
    model = LlamaForCausalLM.random_init(LlamaConfig(**meta["config"]),
                                         ExtraModelConfig(interleave_rope=False, max_len_override=8, max_batch_size=96), seed=1)
    with pytest.raises(AssertionError):
        ThroughputScheduleBuilder.build(model)


def test_oracle_reproduces_the_reference_bit_for_bit():
    from oracle import pyvm_throughput
    from thor_megakernels_b200.demos.throughput.scheduler import ThroughputScheduleBuilder

    meta, arrays, model = build_tiny()
    assert meta["oracle_bit_identical"]
    sched = ThroughputScheduleBuilder.build(model)
    load_inputs(sched, model, meta, arrays)
    pyvm_throughput.interpret_with_pyvm(sched.globs, sched.get_linear_instructions())
    for name in ("hidden_states", "rms_rope_intermediates", "post_ln_rope_q", "attn_out", "rms_gate_intermediates", "silu_out",
                 "rms_lm_head_intermediates", "logits"):
        assert torch.equal(getattr(sched.globs, name), bf16_from_u16(arrays[name])), name
    pos = meta["pos_id"]
    assert torch.equal(model.stacked_kv_cache[0][:, :, pos], bf16_from_u16(arrays["k_rows"]))
    assert torch.equal(model.stacked_kv_cache[1][:, :, pos], bf16_from_u16(arrays["v_rows"]))
    assert np.array_equal(sched.globs.barriers.numpy(), arrays["barriers"])


def test_dispatch_maps_hold_both_instruction_sets():
    from thor_megakernels_b200 import dispatch

    assert set(dispatch.BUILDER_MAP) == {"latency", "throughput"} == set(dispatch.MK_INTERPRETER_MAP)
    a, b = dispatch.make_mk_interpreter("latency"), dispatch.make_mk_interpreter("throughput")
    assert a.mk_func is not b.mk_func
