"""Generates the golden vectors under tests/golden/ by running the REFERENCE's
own code (imported unchanged from a checkout of yiannisha/thor-megakernels) on
this repository's seeded weights.

    python tests/golden/make_golden.py --reference /path/to/thor-megakernels [--case tiny|llama1b|llama1b_layers|all]

What is run from the reference: ``LlamaForCausalLM`` (prefill through its
PyTorch forward), ``LatencyScheduleBuilder`` + ``assign_to_sms`` +
``tensorize_instructions``, and ``PyVM_Generator.run`` for every decode step.
Three shims make it importable on a CPU-only box: a stub ``accelerate`` module,
a constant ``get_sm_count`` (148, the B200 SM count), and parameter
initialisers turned into no-ops (all weights are overwritten with this
repository's seeded tensors before use).

While it runs, the script also executes this repository's restatement
(``oracle/pyvm.py``) on identical inputs and records whether every buffer was
bit-identical (``oracle_bit_identical`` in the metadata).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
import time
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))

SM_COUNT = 148


def import_reference(ref_root: Path):
    import transformers  # noqa: F401  (must be imported before the stub below)

    stub = types.ModuleType("accelerate")

    class _Noop:
        def __init__(self, *a, **k):
            pass

        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

    stub.init_empty_weights = _Noop
    sys.modules.setdefault("accelerate", stub)
    sys.path.insert(0, str(ref_root))
    import megakernels.utils as ru

    ru.get_sm_count = lambda device=None: SM_COUNT
    import megakernels.instructions as ri

    ri.get_sm_count = ru.get_sm_count
    import megakernels.demos.latency.scheduler as rs

    rs.get_sm_count = ru.get_sm_count
    return ru


def u16(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit pattern (numpy has no bf16)."""
    return t.detach().contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def sha(t: torch.Tensor) -> str:
    raw = t.detach().contiguous()
    if raw.dtype == torch.bfloat16:
        raw = raw.view(torch.int16)
    return hashlib.sha256(raw.numpy().tobytes()).hexdigest()


def build_pair(cfg_kwargs: dict, max_len: int, seed: int):
    """This repository's model and the reference's model holding the same weights."""
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig

    mine = LlamaForCausalLM.random_init(
        LlamaConfig(**cfg_kwargs), ExtraModelConfig(interleave_rope=True, max_len_override=max_len), seed=seed,
        finalize=False,
    )

    from megakernels.llama import LlamaForCausalLM as RefLM
    from megakernels.model_types import ExtraModelConfig as RefExtra
    from transformers import LlamaConfig as HFConfig

    c = mine.config
    hf = HFConfig(
        hidden_size=c.hidden_size, intermediate_size=c.intermediate_size, num_hidden_layers=c.num_hidden_layers,
        num_attention_heads=c.num_attention_heads, num_key_value_heads=c.num_key_value_heads, head_dim=c.head_dim,
        vocab_size=c.vocab_size, rms_norm_eps=c.rms_norm_eps, rope_theta=c.rope_theta,
        max_position_embeddings=c.max_position_embeddings, tie_word_embeddings=c.tie_word_embeddings,
        rope_scaling=dict(c.rope_scaling),
    )
    saved = (torch.nn.Linear.reset_parameters, torch.nn.Embedding.reset_parameters)
    torch.nn.Linear.reset_parameters = lambda self: None
    torch.nn.Embedding.reset_parameters = lambda self: None
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        ref = RefLM(hf, RefExtra(interleave_rope=True, max_len_override=max_len))
    finally:
        torch.set_default_dtype(prev)
        torch.nn.Linear.reset_parameters, torch.nn.Embedding.reset_parameters = saved
    ref.requires_grad_(False)

    with torch.no_grad():
        ref.model.embed_tokens.embed_tokens.weight.copy_(mine.model.embed_tokens.embed_tokens.weight)
        for rl, ml in zip(ref.model.layers, mine.model.layers):
            for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
                getattr(rl.self_attn, name).weight.copy_(getattr(ml.self_attn, name).weight)
            for name in ("up_proj", "gate_proj", "down_proj"):
                getattr(rl.mlp, name).weight.copy_(getattr(ml.mlp, name).weight)
            rl.self_attn.input_layernorm.weight.fill_(1.0)
            rl.mlp.input_layernorm.weight.fill_(1.0)
        ref.lm_head.input_norm.weight.fill_(1.0)
        if c.tie_word_embeddings:
            ref.lm_head.lm_head.weight = ref.model.embed_tokens.embed_tokens.weight
        else:
            ref.lm_head.lm_head.weight.copy_(mine.lm_head.lm_head.weight)
    # what from_pretrained does after loading (reference llama.py:632-636)
    ref.model.interleave_rope()
    ref.stack_params()
    ref.setup_caches()
    mine.finalize()
    return mine, ref


def run_case(name: str, cfg_kwargs: dict, max_len: int, prompt_len: int, ntok: int, full_logit_steps, kv_steps,
             keep_all_buffers: bool):
    from megakernels.demos.latency.python_vm import INSTRUCTION_TO_SOLVER as REF_SOLVERS
    from megakernels.demos.latency.scheduler import LatencyScheduleBuilder as RefBuilder
    from megakernels.generators import PyVM_Generator as RefPyVMGen
    from megakernels.model_types import BatchState as RefBatch
    from megakernels.python_vm import PyVM_Interpreter as RefPyVM
    from megakernels.scheduler import assign_to_sms as ref_assign, tensorize_instructions as ref_tensorize

    from oracle import pyvm as mine_vm
    from thor_megakernels_b200.demos.latency.scheduler import LatencyScheduleBuilder
    from thor_megakernels_b200.model_types import BatchState
    from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    t0 = time.time()
    mine, ref = build_pair(cfg_kwargs, max_len, seed=0)
    print(f"[{name}] models built in {time.time() - t0:.1f}s", flush=True)

    meta: dict = {"case": name, "config": cfg_kwargs, "max_len": max_len, "prompt_len": prompt_len, "ntok": ntok,
                  "sm_count": SM_COUNT, "torch": torch.__version__,
                  "cpu_capability": torch.backends.cpu.get_cpu_capability()}
    arrays: dict[str, np.ndarray] = {}

    # ---- model container parity: stacked weights and rotary tables ----
    pairs = {
        "qkv_proj": (mine.stacked_params.qkv_proj, ref.stacked_params.qkv_proj),
        "o_proj": (mine.stacked_params.o_proj, ref.stacked_params.o_proj),
        "up_proj": (mine.stacked_params.up_proj, ref.stacked_params.up_proj),
        "gate_proj": (mine.stacked_params.gate_proj, ref.stacked_params.gate_proj),
        "down_proj": (mine.stacked_params.down_proj, ref.stacked_params.down_proj),
        "lm_head": (mine.lm_head.lm_head.weight, ref.lm_head.lm_head.weight),
    }
    meta["weights_sha256"] = {}
    for k, (a, b) in pairs.items():
        assert torch.equal(a, b), f"stacked {k} differs from the reference's"
        meta["weights_sha256"][k] = sha(b)
    n_rope = mine.model.rope_cos.shape[0]
    assert torch.equal(mine.model.rope_cos, ref.model.rope_cos[:n_rope]), "rope_cos differs from the reference's"
    assert torch.equal(mine.model.rope_sin, ref.model.rope_sin[:n_rope]), "rope_sin differs from the reference's"
    meta["rope_sha256"] = {"cos": sha(ref.model.rope_cos[:n_rope]), "sin": sha(ref.model.rope_sin[:n_rope])}

    # ---- schedule parity ----
    ref_sched = RefBuilder.build(ref)
    my_sched = LatencyScheduleBuilder.build(mine)
    meta["instructions_sha256"] = {}
    for mode in ("rr", "zz", "wave", "dag"):
        ref_tensorize(ref_sched.globs, ref_assign(mode, schedule=ref_sched))
        tensorize_instructions(my_sched.globs, assign_to_sms(mode, schedule=my_sched))
        assert torch.equal(ref_sched.globs.instructions, my_sched.globs.instructions), f"{mode} queues differ"
        meta["instructions_sha256"][mode] = sha(ref_sched.globs.instructions)
        meta.setdefault("instructions_shape", {})[mode] = list(ref_sched.globs.instructions.shape)
    ref_tensorize(ref_sched.globs, ref_assign("rr", schedule=ref_sched))
    tensorize_instructions(my_sched.globs, assign_to_sms("rr", schedule=my_sched))
    meta["dag_nodes"] = len(ref_sched.dag_nodes)
    if keep_all_buffers:
        arrays["instructions_rr"] = ref_sched.globs.instructions.numpy().copy()

    # ---- prompt + prefill through the reference's PyTorch forward ----
    prompt = torch.randint(0, cfg_kwargs["vocab_size"], (1, prompt_len), generator=torch.Generator().manual_seed(1))
    pos = torch.arange(prompt_len)[None]
    out = ref(RefBatch(input_ids=prompt, position_ids=pos, seq_len=prompt_len))
    my_out = mine(BatchState(input_ids=prompt, position_ids=pos, seq_len=prompt_len))
    assert torch.equal(out.output_ids, my_out.output_ids), "prefill tokens differ from the reference's"
    for a, b in zip(mine.stacked_kv_cache, ref.stacked_kv_cache):
        assert torch.equal(a, b), "prefill KV differs from the reference's"
    first = out.output_ids[:, -1:]
    arrays["prompt"] = prompt.numpy().astype(np.int32)
    arrays["prefill_k"] = u16(ref.stacked_kv_cache[0][:, 0, :prompt_len])
    arrays["prefill_v"] = u16(ref.stacked_kv_cache[1][:, 0, :prompt_len])

    # ---- decode with the reference's PyVM generator, oracle in lock step ----
    gen = RefPyVMGen(ref, RefPyVM(REF_SOLVERS), ref_sched)
    my_instr = my_sched.get_linear_instructions()
    tokens = [int(first)]
    hidden, top_idx, top_val, sample_val, margins, step_times = [], [], [], [], [], []
    rng = np.random.default_rng(7)
    sample_idx = np.sort(rng.choice(cfg_kwargs["vocab_size"], size=min(256, cfg_kwargs["vocab_size"]), replace=False))
    arrays["logit_sample_idx"] = sample_idx.astype(np.int32)
    identical = True
    g = ref_sched.globs
    names = ("hidden_states", "post_ln_rope_q", "attn_out", "silu_out", "logits", "barriers")
    for step in range(ntok):
        pos_id = prompt_len + step
        inp = torch.tensor([[tokens[-1]]])
        ts = time.time()
        nxt = gen.run(inp, pos_id=pos_id)
        step_times.append(time.time() - ts)
        my_next = mine_vm.pyvm_step(mine, my_sched, my_instr, inp, pos_id)
        same = int(nxt) == int(my_next)
        for n in names:
            same &= torch.equal(getattr(g, n), getattr(my_sched.globs, n))
        same &= torch.equal(ref.stacked_kv_cache[0][:, 0, pos_id], mine.stacked_kv_cache[0][:, 0, pos_id])
        same &= torch.equal(ref.stacked_kv_cache[1][:, 0, pos_id], mine.stacked_kv_cache[1][:, 0, pos_id])
        identical &= bool(same)
        tokens.append(int(nxt))
        hidden.append(u16(g.hidden_states))
        lf = g.logits.float()
        tv, ti = torch.topk(lf, 8)
        top_idx.append(ti.numpy().astype(np.int32))
        top_val.append(u16(g.logits[ti]))
        sample_val.append(u16(g.logits[torch.from_numpy(sample_idx).long()]))
        margins.append(float(tv[0] - tv[1]))
        if step in full_logit_steps:
            arrays[f"logits_step{step}"] = u16(g.logits)
        if step in kv_steps:
            arrays[f"k_row_step{step}"] = u16(ref.stacked_kv_cache[0][:, 0, pos_id])
            arrays[f"v_row_step{step}"] = u16(ref.stacked_kv_cache[1][:, 0, pos_id])
        if keep_all_buffers:
            arrays[f"q_step{step}"] = u16(g.post_ln_rope_q)
            arrays[f"attn_out_step{step}"] = u16(g.attn_out)
            arrays[f"silu_out_step{step}"] = u16(g.silu_out)
            arrays[f"barriers_step{step}"] = g.barriers.numpy().astype(np.int32).copy()
        if step % 10 == 0:
            print(f"[{name}] step {step} token {tokens[-1]} margin {margins[-1]:.4f} "
                  f"identical={identical} {step_times[-1]:.2f}s", flush=True)
    arrays["tokens"] = np.asarray(tokens, dtype=np.int32)
    arrays["hidden"] = np.stack(hidden)
    arrays["top8_idx"] = np.stack(top_idx)
    arrays["top8_val"] = np.stack(top_val)
    arrays["logit_sample_val"] = np.stack(sample_val)
    arrays["top2_margin"] = np.asarray(margins, dtype=np.float32)
    arrays["last_layer_k_rows"] = u16(ref.stacked_kv_cache[0][-1, 0, prompt_len : prompt_len + ntok])
    arrays["last_layer_v_rows"] = u16(ref.stacked_kv_cache[1][-1, 0, prompt_len : prompt_len + ntok])
    meta["oracle_bit_identical"] = bool(identical)
    meta["reference_pyvm_seconds_per_token"] = float(np.median(step_times))
    meta["cpu_threads"] = torch.get_num_threads()
    assert identical, "oracle/pyvm.py is not bit-identical to the reference's python_vm on this machine"

    np.savez_compressed(HERE / f"{name}.npz", **arrays)
    (HERE / f"{name}.json").write_text(json.dumps(meta, indent=1))
    print(f"[{name}] wrote {name}.npz ({(HERE / (name + '.npz')).stat().st_size / 1e6:.2f} MB), "
          f"oracle identical: {identical}", flush=True)


def run_layers_case(name: str, cfg_kwargs: dict, max_len: int, prompt_len: int, steps: int):
    """Per-layer record of the reference interpreter's residual stream: for each
    of the first ``steps`` decode steps, the hidden state entering every layer,
    the layer's q / attn_out / silu_out, its output and its appended K/V rows.
    A layer can then be run alone from the reference's own input, which pins it
    at the stated tolerance without the rounding noise of the layers before it."""
    from megakernels.demos.latency.python_vm import INSTRUCTION_TO_SOLVER as REF_SOLVERS
    from megakernels.demos.latency.scheduler import LatencyScheduleBuilder as RefBuilder
    from megakernels.model_types import BatchState as RefBatch
    from megakernels.python_vm import interpret_with_pyvm as ref_interpret

    from oracle import pyvm as mine_vm
    from thor_megakernels_b200.demos.latency.scheduler import LatencyScheduleBuilder
    from thor_megakernels_b200.model_types import BatchState

    mine, ref = build_pair(cfg_kwargs, max_len, seed=0)
    ref_sched = RefBuilder.build(ref)
    my_sched = LatencyScheduleBuilder.build(mine)
    prompt = torch.randint(0, cfg_kwargs["vocab_size"], (1, prompt_len), generator=torch.Generator().manual_seed(1))
    pos = torch.arange(prompt_len)[None]
    out = ref(RefBatch(input_ids=prompt, position_ids=pos, seq_len=prompt_len))
    mine(BatchState(input_ids=prompt, position_ids=pos, seq_len=prompt_len))
    token = int(out.output_ids[:, -1])
    g, mg = ref_sched.globs, my_sched.globs
    layers = cfg_kwargs["num_hidden_layers"]
    by_layer = [[] for _ in range(layers)]
    tail = []
    for ins in ref_sched.get_linear_instructions():
        (by_layer[ins.layer_idx] if hasattr(ins, "layer_idx") else tail).append(ins)
    my_by_layer = [[] for _ in range(layers)]
    my_tail = []
    for ins in my_sched.get_linear_instructions():
        (my_by_layer[ins.layer_idx] if hasattr(ins, "layer_idx") else my_tail).append(ins)
    arrays = {"prefill_k": u16(ref.stacked_kv_cache[0][:, 0, :prompt_len]),
              "prefill_v": u16(ref.stacked_kv_cache[1][:, 0, :prompt_len])}
    tokens, identical = [token], True
    keep = {k: [] for k in ("layer_in", "q", "attn_out", "silu_out", "layer_out", "k_rows", "v_rows")}
    for step in range(steps):
        pos_id = prompt_len + step
        inp = torch.tensor([[tokens[-1]]])
        emb = ref.model.embed_tokens(RefBatch(input_ids=inp))
        g.hidden_states[:] = emb.hidden_states
        g.barriers.zero_()
        g.pos_id = pos_id
        mg.hidden_states[:] = mine.model.embed_tokens(BatchState(input_ids=inp)).hidden_states
        mg.barriers.zero_()
        mg.pos_id = pos_id
        rec = {k: [] for k in keep}
        for layer in range(layers):
            rec["layer_in"].append(u16(g.hidden_states))
            ref_interpret(g, by_layer[layer], REF_SOLVERS)
            mine_vm.interpret_with_pyvm(mg, my_by_layer[layer])
            for n in ("hidden_states", "post_ln_rope_q", "attn_out", "silu_out"):
                identical &= torch.equal(getattr(g, n), getattr(mg, n))
            rec["q"].append(u16(g.post_ln_rope_q))
            rec["attn_out"].append(u16(g.attn_out))
            rec["silu_out"].append(u16(g.silu_out))
            rec["layer_out"].append(u16(g.hidden_states))
            rec["k_rows"].append(u16(ref.stacked_kv_cache[0][layer, 0, pos_id]))
            rec["v_rows"].append(u16(ref.stacked_kv_cache[1][layer, 0, pos_id]))
        ref_interpret(g, tail, REF_SOLVERS)
        emb.hidden_states = g.hidden_states
        tokens.append(int(ref.lm_head(emb).output_ids))
        for k in keep:
            keep[k].append(np.stack(rec[k]))
        print(f"[{name}] step {step} token {tokens[-1]} identical={identical}", flush=True)
    for k in keep:
        arrays[k] = np.stack(keep[k])   # [steps, layers, ...]
    arrays["tokens"] = np.asarray(tokens, dtype=np.int32)
    assert identical, "oracle/pyvm.py is not bit-identical to the reference's python_vm, layer by layer"
    meta = {"case": name, "config": cfg_kwargs, "max_len": max_len, "prompt_len": prompt_len, "steps": steps,
            "oracle_bit_identical": bool(identical), "torch": torch.__version__}
    np.savez_compressed(HERE / f"{name}.npz", **arrays)
    (HERE / f"{name}.json").write_text(json.dumps(meta, indent=1))
    print(f"[{name}] wrote {name}.npz ({(HERE / (name + '.npz')).stat().st_size / 1e6:.2f} MB)", flush=True)


CASES = {
    # two layers, small vocabulary: every buffer of every step is kept
    "tiny": dict(cfg_kwargs=dict(hidden_size=2048, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8,
                                 head_dim=64, intermediate_size=8192, vocab_size=4096), max_len=64, prompt_len=8,
                 ntok=4, full_logit_steps=(0, 1, 2, 3), kv_steps=(0, 1, 2, 3), keep_all_buffers=True),
    # Llama-3.2-1B architecture, 16-token prompt, 100 greedy tokens
    "llama1b": dict(cfg_kwargs=dict(hidden_size=2048, num_hidden_layers=16, num_attention_heads=32,
                                    num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=128256),
                    max_len=256, prompt_len=16, ntok=100, full_logit_steps=(0, 50, 99), kv_steps=(0, 50, 99),
                    keep_all_buffers=False),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, required=True)
    ap.add_argument("--case", default="all")
    args = ap.parse_args()
    import_reference(args.reference)
    torch.set_grad_enabled(False)
    for name, spec in CASES.items():
        if args.case in ("all", name):
            run_case(name, **spec)
    if args.case in ("all", "llama1b_layers"):
        # same model, prompt and token stream as the llama1b case
        spec = CASES["llama1b"]
        run_layers_case("llama1b_layers", spec["cfg_kwargs"], spec["max_len"], spec["prompt_len"], steps=3)


if __name__ == "__main__":
    main()
