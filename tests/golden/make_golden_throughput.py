"""Pins the batched instruction set against the REFERENCE (imported unchanged
from a checkout of yiannisha/thor-megakernels):

    python tests/golden/make_golden_throughput.py --reference /path/to/thor-megakernels

A small model (2 layers, hidden 512, batch 128) with this repository's seeded
weights is run through the reference's ThroughputScheduleBuilder and its
throughput python_vm for one decode step; this repository's builder and
oracle/pyvm_throughput.py run beside it and every instruction tensor and every
buffer must be bit-identical.  Buffers go to tests/golden/throughput_tiny.npz.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(HERE))

CFG = dict(hidden_size=512, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
           intermediate_size=768, vocab_size=384)
BATCH, MAX_LEN, POS = 128, 12, 9


def main():
    from make_golden import import_reference, sha, u16

    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, required=True)
    args = ap.parse_args()
    import_reference(args.reference)
    torch.set_grad_enabled(False)

    from megakernels.demos.throughput.python_vm import INSTRUCTION_TO_SOLVER as REF_SOLVERS
    from megakernels.demos.throughput.scheduler import ThroughputScheduleBuilder as RefBuilder
    from megakernels.llama import LlamaForCausalLM as RefLM
    from megakernels.model_types import ExtraModelConfig as RefExtra
    from megakernels.python_vm import interpret_with_pyvm as ref_interpret
    from megakernels.scheduler import assign_to_sms as ref_assign, tensorize_instructions as ref_tensorize
    from transformers import LlamaConfig as HFConfig

    from oracle import pyvm_throughput
    from thor_megakernels_b200.demos.throughput.scheduler import ThroughputScheduleBuilder
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig
    from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    mine = LlamaForCausalLM.random_init(LlamaConfig(**CFG), ExtraModelConfig(interleave_rope=False, max_len_override=MAX_LEN,
                                                                             max_batch_size=BATCH), seed=5, finalize=False)
    c = mine.config
    hf = HFConfig(hidden_size=c.hidden_size, intermediate_size=c.intermediate_size, num_hidden_layers=c.num_hidden_layers,
                  num_attention_heads=c.num_attention_heads, num_key_value_heads=c.num_key_value_heads, head_dim=c.head_dim,
                  vocab_size=c.vocab_size, rms_norm_eps=c.rms_norm_eps, rope_theta=c.rope_theta,
                  max_position_embeddings=c.max_position_embeddings, tie_word_embeddings=c.tie_word_embeddings,
                  rope_scaling=dict(c.rope_scaling))
    saved = (torch.nn.Linear.reset_parameters, torch.nn.Embedding.reset_parameters)
    torch.nn.Linear.reset_parameters = lambda self: None
    torch.nn.Embedding.reset_parameters = lambda self: None
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        ref = RefLM(hf, RefExtra(interleave_rope=False, max_len_override=MAX_LEN, max_batch_size=BATCH))
    finally:
        torch.set_default_dtype(prev)
        torch.nn.Linear.reset_parameters, torch.nn.Embedding.reset_parameters = saved
    ref.requires_grad_(False)
    ref.model.embed_tokens.embed_tokens.weight.copy_(mine.model.embed_tokens.embed_tokens.weight)
    for rl, ml in zip(ref.model.layers, mine.model.layers):
        for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
            getattr(rl.self_attn, name).weight.copy_(getattr(ml.self_attn, name).weight)
        for name in ("up_proj", "gate_proj", "down_proj"):
            getattr(rl.mlp, name).weight.copy_(getattr(ml.mlp, name).weight)
        rl.self_attn.input_layernorm.weight.fill_(1.0)
        rl.mlp.input_layernorm.weight.fill_(1.0)
    ref.lm_head.input_norm.weight.fill_(1.0)
    ref.lm_head.lm_head.weight = ref.model.embed_tokens.embed_tokens.weight
    ref.stack_params()
    ref.setup_caches()
    mine.finalize()

    ref_sched, my_sched = RefBuilder.build(ref), ThroughputScheduleBuilder.build(mine)
    meta = {"config": CFG, "batch": BATCH, "max_len": MAX_LEN, "pos_id": POS, "dag_nodes": len(ref_sched.dag_nodes),
            "instructions_sha256": {}}
    for mode, kw in (("rr", {}), ("zz", {}), ("pool", dict(memory_fraction=0.5))):
        ref_tensorize(ref_sched.globs, ref_assign(mode, schedule=ref_sched, **kw))
        tensorize_instructions(my_sched.globs, assign_to_sms(mode, schedule=my_sched, **kw))
        assert torch.equal(ref_sched.globs.instructions, my_sched.globs.instructions), f"{mode} queues differ"
        meta["instructions_sha256"][mode] = sha(ref_sched.globs.instructions)

    gen = torch.Generator().manual_seed(17)
    hidden = torch.randn(BATCH, CFG["hidden_size"], generator=gen).bfloat16()
    kv = [torch.randn(ref.stacked_kv_cache[i].shape, generator=gen).bfloat16() for i in range(2)]
    for g, model in ((ref_sched.globs, ref), (my_sched.globs, mine)):
        g.hidden_states[:] = hidden
        g.pos_id = POS
        g.barriers.zero_()
        for i in range(2):
            model.stacked_kv_cache[i].copy_(kv[i])
    ref_interpret(ref_sched.globs, ref_sched.get_linear_instructions(), REF_SOLVERS)
    pyvm_throughput.interpret_with_pyvm(my_sched.globs, my_sched.get_linear_instructions())
    names = ("hidden_states", "rms_rope_intermediates", "post_ln_rope_q", "attn_out", "rms_gate_intermediates", "silu_out",
             "rms_lm_head_intermediates", "logits")
    arrays = {"hidden_in": u16(hidden), "k_in": u16(kv[0]), "v_in": u16(kv[1])}
    identical = True
    for n in names:
        identical &= torch.equal(getattr(ref_sched.globs, n), getattr(my_sched.globs, n))
        arrays[n] = u16(getattr(ref_sched.globs, n))
    identical &= torch.equal(ref_sched.globs.barriers, my_sched.globs.barriers)
    for i, name in enumerate(("k_rows", "v_rows")):
        identical &= torch.equal(ref.stacked_kv_cache[i][:, :, POS], mine.stacked_kv_cache[i][:, :, POS])
        arrays[name] = u16(ref.stacked_kv_cache[i][:, :, POS])
    arrays["barriers"] = ref_sched.globs.barriers.numpy().astype(np.int32)
    meta["oracle_bit_identical"] = bool(identical)
    assert identical, "oracle/pyvm_throughput.py is not bit-identical to the reference's throughput python_vm"
    np.savez_compressed(HERE / "throughput_tiny.npz", **arrays)
    (HERE / "throughput_tiny.json").write_text(json.dumps(meta, indent=1))
    print("wrote throughput_tiny.npz", (HERE / "throughput_tiny.npz").stat().st_size, "bytes; identical:", identical)


if __name__ == "__main__":
    main()
