"""GPU parity of the kernel paths that the larger workloads run, each against
the CPU oracle (never against another GPU path), through the C-ABI library:

* every layer of the Llama-3.2-1B architecture alone, fed the reference
  interpreter's own residual stream (tests/golden/llama1b_layers.npz), at the
  stated tolerance ``|a - ref| <= 3e-2 + 1e-2 |ref|``;
* 128-wide heads with the cache split into 8 and 24 slices plus the
  log-sum-exp merge (the Llama-3.1-8B attention path at long context);
* NVFP4 weight-only models at hidden size 4096, with split attention at 4096
  cached positions, and on tensor-parallel shard shapes;
* a non-terminal attention merge.
"""
import numpy as np
import pytest
import torch

from helpers import assert_close, bf16_from_u16, build_model, build_schedule, load_golden

pytestmark = pytest.mark.gpu

B1 = dict(hidden_size=2048, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
          intermediate_size=8192, vocab_size=4096)
B8 = dict(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
          intermediate_size=14336, vocab_size=4096, tie_word_embeddings=False,
          rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                            original_max_position_embeddings=8192))


# ---------------------------------------------------------------------------
# every layer of the 1B model, teacher-forced on the reference's residual stream
# ---------------------------------------------------------------------------

def test_llama1b_every_layer_alone_from_the_reference_residual_stream():
    """Layer l of the 16-layer model is run by itself: its input is the hidden
    state the reference interpreter had when it entered layer l, and the cache
    holds the reference's rows for all earlier positions.  Nothing upstream of
    the layer is computed on the GPU, so no rounding noise has been amplified
    and every buffer must meet the element-wise band.  Steps 0, 1 and 2 of the
    100-token request (positions 16, 17, 18)."""
    from thor_megakernels_b200.runtime import Megakernel

    meta, arrays = load_golden("llama1b_layers")
    cfg, n = meta["config"], meta["prompt_len"]
    layers = cfg["num_hidden_layers"]
    model = build_model(cfg, meta["max_len"], device="cuda")
    k_cache, v_cache = model.stacked_kv_cache
    k_cache[:, 0, :n] = bf16_from_u16(arrays["prefill_k"]).cuda()
    v_cache[:, 0, :n] = bf16_from_u16(arrays["prefill_v"]).cuda()
    # one handle on one set of activation buffers; only the instruction queues change from layer to layer
    scheds = [build_schedule(model, first_layer=layer, layer_limit=layer + 1) for layer in range(layers)]
    g = scheds[0].globs
    mk = Megakernel.from_globals(g)
    worst = {}
    for step in range(meta["steps"]):
        pos = n + step
        for layer in range(layers):
            mk.set_schedule(scheds[layer].globs.instructions, scheds[layer].globs.timings)
            g.hidden_states[:] = bf16_from_u16(arrays["layer_in"][step, layer]).cuda()
            g.barriers.zero_()
            mk.step(pos)
            assert mk.status()["code"] == 0
            checks = {
                "q": (g.post_ln_rope_q, arrays["q"]), "attn_out": (g.attn_out, arrays["attn_out"]),
                "silu_out": (g.silu_out, arrays["silu_out"]), "layer_out": (g.hidden_states, arrays["layer_out"]),
                "k_row": (k_cache[layer, 0, pos], arrays["k_rows"]), "v_row": (v_cache[layer, 0, pos], arrays["v_rows"]),
            }
            for name, (got, ref) in checks.items():
                rep = assert_close(f"step {step} layer {layer} {name}", got, bf16_from_u16(ref[step, layer]))
                worst[name] = max(worst.get(name, 0.0), rep["max_abs"])
        # the next step's cache is the reference's, not what the GPU appended
        k_cache[:, 0, pos] = bf16_from_u16(arrays["k_rows"][step]).cuda().view(layers, -1, cfg["head_dim"])
        v_cache[:, 0, pos] = bf16_from_u16(arrays["v_rows"][step]).cuda().view(layers, -1, cfg["head_dim"])
    print("worst max-abs per buffer over 3 steps x 16 layers:", {k: round(v, 4) for k, v in worst.items()})


# ---------------------------------------------------------------------------
# 128-wide heads, split cache + merge
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("partitions,context", [(8, 1024), (24, 1500), (18, 2111), (4, 2111), (2, 1500)])
def test_split_attention_128_wide_heads(partitions, context):
    """The attention path of the 8B shapes at long context: cache split over
    several CTAs per KV head, 128-wide heads, log-sum-exp merge; seeded N(0,1)
    keys/values and std-100 garbage beyond the context."""
    from oracle import pyvm
    from thor_megakernels_b200.dispatch import make_mk_interpreter

    max_len = 2304
    cpu_model = build_model(B8, max_len, device="cpu", seed=4)
    model = build_model(B8, max_len, device="cuda", seed=4)
    gen = torch.Generator().manual_seed(17)
    for idx in range(2):
        kv = torch.randn(cpu_model.stacked_kv_cache[idx].shape, generator=gen).bfloat16()
        kv[:, :, context:] *= 100.0
        cpu_model.stacked_kv_cache[idx].copy_(kv)
        model.stacked_kv_cache[idx].copy_(kv.cuda())
    h0 = torch.randn(B8["hidden_size"], generator=gen).bfloat16()
    kwargs = dict(skip_attn_reduction=False, num_attention_partitions=partitions, stop_after_op="oproj", layer_limit=1)
    cpu_sched, sched = build_schedule(cpu_model, **kwargs), build_schedule(model, **kwargs)
    for s, dev in ((cpu_sched, "cpu"), (sched, "cuda")):
        s.globs.hidden_states[:] = h0.to(dev)
        s.globs.barriers.zero_()
        s.globs.pos_id = context
    pyvm.interpret_with_pyvm(cpu_sched.globs, cpu_sched.get_linear_instructions())
    make_mk_interpreter("latency").interpret(sched.globs)
    torch.cuda.synchronize()
    assert_close("attn_out", sched.globs.attn_out, cpu_sched.globs.attn_out)
    assert_close("hidden_states", sched.globs.hidden_states, cpu_sched.globs.hidden_states)
    lse_g = sched.globs.attn_lse_intermediates[:, :partitions].cpu()
    lse_c = cpu_sched.globs.attn_lse_intermediates[:, :partitions]
    assert torch.allclose(lse_g, lse_c, atol=1e-3, rtol=1e-4)
    out_g = sched.globs.attn_out_intermediates[:, :partitions].cpu()
    out_c = cpu_sched.globs.attn_out_intermediates[:, :partitions]
    assert torch.allclose(out_g, out_c, atol=2e-3, rtol=1e-3)
    assert torch.equal(sched.globs.barriers.cpu()[:, :6], cpu_sched.globs.barriers[:, :6])


def test_non_terminal_attention_merge():
    """A merge that is not the last level writes its result back as a new
    partial (here slot 5).  The reference interpreter raises on this branch (it
    assigns a [4, 1] tensor to a [4] slice, latency/python_vm.py:381-387, and no
    reference schedule emits it), so the expected values are the formula it
    spells out, evaluated on the oracle's partials: weights exp2(lse - max),
    weighted mean of the partial outputs, natural log of the weight sum."""
    from oracle import pyvm
    from thor_megakernels_b200.demos.latency.instructions import AttentionReduction
    from thor_megakernels_b200.dispatch import make_mk_interpreter
    from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    cpu_model = build_model(B1, 256, device="cpu", seed=3)
    model = build_model(B1, 256, device="cuda", seed=3)
    gen = torch.Generator().manual_seed(23)
    context = 130
    for idx in range(2):
        kv = torch.randn(cpu_model.stacked_kv_cache[idx].shape, generator=gen).bfloat16()
        cpu_model.stacked_kv_cache[idx].copy_(kv)
        model.stacked_kv_cache[idx].copy_(kv.cuda())
    h0 = torch.randn(B1["hidden_size"], generator=gen).bfloat16()
    kwargs = dict(skip_attn_reduction=False, num_attention_partitions=4, stop_after_op="partial", layer_limit=1)
    cpu_sched, sched = build_schedule(cpu_model, **kwargs), build_schedule(model, **kwargs)
    merges = [AttentionReduction(layer_idx=0, head_start_idx=4 * kv_head, num_partials=4, is_terminal=False,
                                 reduction_list=[0, 1, 2, 3], output_partial_idx=5) for kv_head in range(8)]
    tensorize_instructions(sched.globs, assign_to_sms("rr", instructions=sched.get_linear_instructions() + merges,
                                                      sm_count=sched.globs.sm_count()))
    for s, dev in ((cpu_sched, "cpu"), (sched, "cuda")):
        s.globs.hidden_states[:] = h0.to(dev)
        s.globs.barriers.zero_()
        s.globs.pos_id = context
    pyvm.interpret_with_pyvm(cpu_sched.globs, cpu_sched.get_linear_instructions())
    make_mk_interpreter("latency").interpret(sched.globs)
    torch.cuda.synchronize()
    g, c = sched.globs, cpu_sched.globs
    lses, outs = c.attn_lse_intermediates[:, :4], c.attn_out_intermediates[:, :4]
    weights = (lses - lses.max(dim=-1, keepdim=True).values).exp2()
    want_out = (outs * weights.unsqueeze(-1)).sum(dim=1) / weights.sum(dim=-1, keepdim=True)
    want_lse = weights.sum(dim=-1).log()
    assert torch.allclose(g.attn_lse_intermediates[:, :4].cpu(), lses, atol=1e-3, rtol=1e-4)
    assert torch.allclose(g.attn_lse_intermediates[:, 5].cpu(), want_lse, atol=1e-3, rtol=1e-4)
    assert torch.allclose(g.attn_out_intermediates[:, 5].cpu(), want_out, atol=2e-3, rtol=1e-3)
    # counters: the partials' row as in the interpreter, plus 4 heads per merge in the merge row
    assert torch.equal(g.barriers.cpu()[:, :2], c.barriers[:, :2])
    assert int(g.barriers[0, 2, 0]) == 32


# ---------------------------------------------------------------------------
# NVFP4 weight-only models
# ---------------------------------------------------------------------------

def _oracle_weights(q, layers):
    """The oracle decodes exactly the bytes the device quantiser produced (those
    are checked bit for bit against the oracle quantiser in test_gpu_nvfp4.py)."""
    from oracle import nvfp4 as fmt, nvfp4_model

    def to_oracle(w):
        dq = fmt.dequantize(w.packed.cpu().numpy(), w.scales.cpu().numpy(), w.tensor_scale)
        return nvfp4_model.QuantMatrix(None, None, np.float32(w.tensor_scale), torch.from_numpy(dq))

    per_layer = [nvfp4_model.QuantLayer(*(to_oracle(q[k][i]) for k in ("qkv", "o", "up", "gate", "down")))
                 for i in range(layers)]
    return per_layer, to_oracle(q["lm_head"])


class _exact_linears:
    """While active, the quantised-model oracle's linears accumulate in float64
    and round once: what any summation order gives with perfect accumulation."""

    def __enter__(self):
        from oracle import nvfp4_model

        self._mod, self._plain = nvfp4_model, nvfp4_model._linear
        nvfp4_model._linear = lambda x, q: (x.double() @ q.dequant.double().T).bfloat16()
        return self

    def __exit__(self, *exc):
        self._mod._linear = self._plain
        return False


def _nvfp4_steps(cpu, gpu, ctx, steps, first_token=77, partitions=1, check=("silu_out", "attn_out"), exact=None):
    """Decode ``steps`` tokens with NVFP4 weight-only linears on the GPU and in
    the CPU oracle, teacher-forced on the oracle's tokens.  Every buffer must
    meet |a - ref| <= 3e-2 + 1e-2 |ref|.  With ``exact`` (a second CPU copy of the
    model): where 4096-wide sums push even an exactly accumulated restatement
    out of that band after two layers, at most twice that restatement's own
    distance from the oracle (helpers.assert_parity)."""
    from helpers import assert_parity
    from oracle import nvfp4_model
    from thor_megakernels_b200.nvfp4 import quantize_model
    from thor_megakernels_b200.runtime import MK_STEP_EMBED, MK_STEP_RESET_BARRIERS, MK_STEP_WRITE_TOKEN, Megakernel

    q = quantize_model(gpu)
    layers, head = _oracle_weights(q, gpu.config.num_hidden_layers)
    sched = build_schedule(gpu, skip_attn_reduction=partitions == 1, num_attention_partitions=partitions)
    g = sched.globs
    emb = gpu.model.embed_tokens.embed_tokens.weight.data
    mk = Megakernel.from_globals(g, embed_w=emb, quantized=q)
    tok_in = torch.zeros(1, dtype=torch.int32, device="cuda")
    tok_out = torch.zeros(1, dtype=torch.int32, device="cuda")
    g.barriers.zero_()
    token = first_token
    for step in range(steps):
        pos = ctx + step
        emb_row = cpu.model.embed_tokens.embed_tokens.weight[token]
        hidden, logits, last = nvfp4_model.decode_step(cpu, layers, head, emb_row, pos)
        tok_in.fill_(token)
        mk.step(pos, flags=MK_STEP_EMBED | MK_STEP_RESET_BARRIERS | MK_STEP_WRITE_TOKEN, token_in=tok_in, token_out=tok_out)
        assert mk.status()["code"] == 0
        # layer 0's appended cache row has seen no accumulated rounding noise: always the plain band
        assert_close("layer-0 k row", gpu.stacked_kv_cache[0][0, 0, pos], cpu.stacked_kv_cache[0][0, 0, pos])
        if exact is None:
            for name in check:
                assert_close(name, getattr(g, name), last[name])
            assert_close("hidden", g.hidden_states, hidden)
            assert_close("logits", g.logits, logits)
            assert_close("k rows", gpu.stacked_kv_cache[0][:, 0, pos], cpu.stacked_kv_cache[0][:, 0, pos])
        else:
            with _exact_linears():
                e_hidden, e_logits, e_last = nvfp4_model.decode_step(exact, layers, head, emb_row, pos)
            n_layers = gpu.config.num_hidden_layers
            for name in check:
                print(assert_parity(name, getattr(g, name), last[name], e_last[name], layers=n_layers))
            print(assert_parity("hidden", g.hidden_states, hidden, e_hidden, layers=n_layers))
            print(assert_parity("logits", g.logits, logits, e_logits, layers=n_layers))
            print(assert_parity("k rows", gpu.stacked_kv_cache[0][:, 0, pos], cpu.stacked_kv_cache[0][:, 0, pos],
                                exact.stacked_kv_cache[0][:, 0, pos], layers=n_layers))
        want = int(logits.float().argmax())
        assert int(tok_out) == int(g.logits.float().argmax()), "in-kernel argmax differs from argmax of the logits it wrote"
        if int(tok_out) != want:
            top2 = torch.topk(logits.float(), 2).values
            assert float(top2[0] - top2[1]) <= 0.125
        token = want
    mk.close()


def _fill_cache(cpu, gpu, ctx, seed, garbage=False):
    gen = torch.Generator().manual_seed(seed)
    for idx in range(2):
        if garbage:
            kv = torch.randn(cpu.stacked_kv_cache[idx].shape, generator=gen).bfloat16()
            kv[:, :, ctx:] *= 100.0
            cpu.stacked_kv_cache[idx].copy_(kv)
            gpu.stacked_kv_cache[idx].copy_(kv.cuda())
        else:
            kv = torch.randn(cpu.stacked_kv_cache[idx][:, :, :ctx].shape, generator=gen).bfloat16()
            cpu.stacked_kv_cache[idx][:, :, :ctx] = kv
            gpu.stacked_kv_cache[idx][:, :, :ctx] = kv.cuda()


def test_nvfp4_hidden_4096_two_layers():
    """Llama-3.1-8B layer shapes with every linear NVFP4 weight-only: the
    two-chunk (K = 4096) NVFP4 tile path, seven down-projection slices."""
    cpu = build_model(B8, 64, device="cpu", seed=4)
    exact = build_model(B8, 64, device="cpu", seed=4)
    gpu = build_model(B8, 64, device="cuda", seed=4)
    _fill_cache(cpu, gpu, 21, seed=31)
    _fill_cache(exact, gpu, 21, seed=31)
    _nvfp4_steps(cpu, gpu, ctx=21, steps=2, exact=exact)


def test_nvfp4_split_attention_at_4096_positions():
    """The long-context NVFP4 workload's path: 4096 cached positions split into
    17 slices per KV head plus the merge, NVFP4 linears around it."""
    ctx = 4096
    cpu = build_model(B1, ctx + 8, device="cpu", seed=5)
    gpu = build_model(B1, ctx + 8, device="cuda", seed=5)
    _fill_cache(cpu, gpu, ctx, seed=33, garbage=True)
    _nvfp4_steps(cpu, gpu, ctx=ctx, steps=2, partitions=17)


@pytest.mark.parametrize("cfg,world", [(B1, 2), (B8, 2), (B8, 8)])
def test_nvfp4_on_tensor_parallel_shard_shapes(cfg, world):
    """A tensor-parallel rank's shard is a narrower model; with NVFP4 weights its
    narrow tiles (output projection input of 512 or 2048 columns, 1792-column
    down-projection slices) go through the NVFP4 consumer."""
    from thor_megakernels_b200.tp import shard_model

    cpu = build_model(cfg, 64, device="cpu", seed=3)
    exact = build_model(cfg, 64, device="cpu", seed=3)
    gpu = build_model(cfg, 64, device="cuda", seed=3)
    _fill_cache(cpu, gpu, 19, seed=21)
    _fill_cache(exact, gpu, 19, seed=21)
    rank = world - 1
    cpu_shard, gpu_shard = shard_model(cpu, rank, world), shard_model(gpu, rank, world)
    wide = cfg["hidden_size"] > 2048
    _nvfp4_steps(cpu_shard, gpu_shard, ctx=19, steps=2, exact=shard_model(exact, rank, world) if wide else None)
