"""The reference's batched ("throughput") instruction set executed on the GPU
through ``make_mk_interpreter("throughput")`` (C-ABI ``mk_throughput_*``)
against golden vectors produced by the reference's own interpreter and against
the oracle restatement on the same seeded inputs.  Tolerance: the stated band
``|a - ref| <= 3e-2 + 1e-2 |ref|`` on bf16 buffers; counters bit-exact."""
import numpy as np
import pytest
import torch

from helpers import assert_close, bf16_from_u16, nrmse
from test_throughput_cpu import build_tiny, load_inputs

pytestmark = pytest.mark.gpu

BUFFERS = ("rms_rope_intermediates", "post_ln_rope_q", "attn_out", "rms_gate_intermediates", "silu_out", "hidden_states",
           "rms_lm_head_intermediates", "logits")


def schedule_for(model, mode="rr", nodes=None, **kw):
    from thor_megakernels_b200.demos.throughput.scheduler import ThroughputScheduleBuilder
    from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    sched = ThroughputScheduleBuilder.build(model)
    if nodes is not None:
        sched.dag_nodes = nodes(sched)
    tensorize_instructions(sched.globs, assign_to_sms(mode, schedule=sched, **kw))
    return sched


@pytest.mark.parametrize("mode,kw", [("rr", {}), ("pool", dict(memory_fraction=0.5))])
def test_tiny_model_matches_the_reference_vectors(mode, kw):
    from thor_megakernels_b200.dispatch import make_mk_interpreter

    meta, arrays, model = build_tiny("cuda")
    sched = schedule_for(model, mode, **kw)
    load_inputs(sched, model, meta, arrays)
    make_mk_interpreter("throughput").interpret(sched.globs)
    torch.cuda.synchronize()
    for name in BUFFERS:
        assert_close(name, getattr(sched.globs, name), bf16_from_u16(arrays[name]))
        assert nrmse(getattr(sched.globs, name), bf16_from_u16(arrays[name])) <= 5e-3, name
    pos = meta["pos_id"]
    assert_close("k rows", model.stacked_kv_cache[0][:, :, pos], bf16_from_u16(arrays["k_rows"]))
    assert_close("v rows", model.stacked_kv_cache[1][:, :, pos], bf16_from_u16(arrays["v_rows"]))
    # rows of the cache the step does not own stay as they were
    assert torch.equal(model.stacked_kv_cache[0][:, :, :pos].cpu(), bf16_from_u16(arrays["k_in"])[:, :, :pos])
    assert np.array_equal(sched.globs.barriers.cpu().numpy(), arrays["barriers"])


def test_llama1b_shapes_two_blocks_against_the_oracle():
    """Two layers with the 1B model's widths, 256 sequences (two 128-sequence blocks), position 37."""
    from oracle import pyvm_throughput
    from thor_megakernels_b200.dispatch import make_mk_interpreter
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig

    cfg = LlamaConfig(hidden_size=2048, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
                      intermediate_size=8192, vocab_size=4096)
    extra = ExtraModelConfig(interleave_rope=False, max_len_override=64, max_batch_size=256)
    pos = 37
    gen = torch.Generator().manual_seed(3)
    hidden = torch.randn(256, 2048, generator=gen).bfloat16()
    results = {}
    for device in ("cpu", "cuda"):
        model = LlamaForCausalLM.random_init(cfg, extra, seed=11, device=device)
        g2 = torch.Generator().manual_seed(4)
        for cache in model.stacked_kv_cache:
            cache.copy_(torch.randn(cache.shape, generator=g2).bfloat16())
        sched = schedule_for(model)
        sched.globs.hidden_states[:] = hidden.to(device)
        sched.globs.pos_id = pos
        if device == "cpu":
            pyvm_throughput.interpret_with_pyvm(sched.globs, sched.get_linear_instructions())
        else:
            make_mk_interpreter("throughput").interpret(sched.globs)
            torch.cuda.synchronize()
        results[device] = (sched.globs, model)
    ref, got = results["cpu"], results["cuda"]
    for name in BUFFERS:
        r, g = getattr(ref[0], name), getattr(got[0], name)
        assert nrmse(g, r) <= 1e-2, (name, nrmse(g, r))
        if name in ("rms_rope_intermediates", "post_ln_rope_q", "attn_out"):
            assert_close(name, g, r)
    for i in range(2):
        assert_close("cache rows", got[1].stacked_kv_cache[i][:, :, pos], ref[1].stacked_kv_cache[i][:, :, pos])
    assert torch.equal(ref[0].barriers, got[0].barriers.cpu())
    assert (got[0].logits.float().argmax(-1).cpu() == ref[0].logits.float().argmax(-1)).float().mean() >= 0.97


def test_partial_schedule_runs_only_its_operators():
    """Layer 0's first three operators: q, the cache rows and attention output are written, the rest is untouched."""
    from thor_megakernels_b200.dispatch import make_mk_interpreter

    meta, arrays, model = build_tiny("cuda")
    sched = schedule_for(model, nodes=lambda s: [n for n in s.dag_nodes
                                                 if getattr(n.instruction, "layer_idx", 1) == 0 and n.instruction.opcode() <= 3])
    load_inputs(sched, model, meta, arrays)
    sched.globs.silu_out.fill_(7.0)
    make_mk_interpreter("throughput").interpret(sched.globs)
    torch.cuda.synchronize()
    g = sched.globs
    assert torch.equal(g.hidden_states.cpu(), bf16_from_u16(arrays["hidden_in"]))
    assert bool((g.silu_out == 7.0).all()) and bool((g.logits == 0).all())
    assert float(g.attn_out.float().abs().max()) > 0
    want = np.zeros_like(arrays["barriers"])
    want[0, :3] = arrays["barriers"][0, :3]
    assert np.array_equal(g.barriers.cpu().numpy(), want)


def test_partial_operator_and_bad_operands_are_refused():
    from thor_megakernels_b200._lib import MegakernelError
    from thor_megakernels_b200.dispatch import make_mk_interpreter

    meta, arrays, model = build_tiny("cuda")
    sched = schedule_for(model, nodes=lambda s: s.dag_nodes[:-1])   # one LM-head block missing
    with pytest.raises(MegakernelError, match="whole"):
        make_mk_interpreter("throughput").interpret(sched.globs)
    sched = schedule_for(model)
    bad = sched.globs.instructions.clone()
    slot = (bad[..., 0] == 2).nonzero()[0]
    bad[slot[0], slot[1], 3] = 99     # QKV block outside the matrix
    sched.globs.instructions = bad
    with pytest.raises(MegakernelError, match="outside the model"):
        make_mk_interpreter("throughput").interpret(sched.globs)
