"""Batched-decode linear on the tcgen05 tensor cores against the oracle for a
dense linear with bf16 operands: ``F.linear(x.float(), w.float()).bfloat16()``
(fp32 accumulation, one rounding), through the C-ABI.  Tolerance: the stated
band ``|a - ref| <= 3e-2 + 1e-2 |ref|`` and relative L2 <= 1e-3."""
import pytest
import torch

from helpers import assert_close, nrmse

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def oracle_linear(w, x):
    return torch.nn.functional.linear(x.float().cpu(), w.float().cpu()).bfloat16().float()


@pytest.mark.parametrize("n,k", [(128, 64), (256, 512), (3072, 2048), (2048, 8192), (128256, 2048), (1000, 2048)])
@pytest.mark.parametrize("batch", [1, 16, 64, 128, 37])
def test_linear_matches_the_oracle(n, k, batch):
    from thor_megakernels_b200 import batched

    gen = torch.Generator(device="cuda").manual_seed(n + k + batch)
    w = (torch.randn(n, k, device="cuda", generator=gen) * 0.02).bfloat16()
    x = torch.randn(batch, k, device="cuda", generator=gen).bfloat16()
    got = batched.linear(w, x)
    batched.check_errors()
    assert got.shape == (batch, n)
    want = oracle_linear(w, x)
    assert rel_l2(got.float().cpu(), want) <= 1e-3
    assert_close("linear", got, want)


@pytest.mark.parametrize("n,k,batch", [(2048, 2048, 64), (2048, 8192, 16), (4096, 14336, 128)])
def test_split_k_partials_add_up(n, k, batch):
    from thor_megakernels_b200 import batched

    gen = torch.Generator(device="cuda").manual_seed(5)
    w = (torch.randn(n, k, device="cuda", generator=gen) * 0.02).bfloat16()
    x = torch.randn(batch, k, device="cuda", generator=gen).bfloat16()
    splits = batched.suggested_splits(n, k)
    assert splits > 1 and (k // 64) % splits == 0
    parts = batched.linear(w, x, splits=splits)
    batched.check_errors()
    assert parts.shape == (splits, batch, n)
    got = parts.sum(dim=0).bfloat16()   # split order
    want = oracle_linear(w, x)
    assert rel_l2(got.float().cpu(), want) <= 1e-3
    assert_close("split-K linear", got, want)


def test_bad_shapes_are_refused():
    from thor_megakernels_b200 import batched
    from thor_megakernels_b200._lib import MegakernelError

    w = torch.zeros(128, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(MegakernelError):
        batched.linear(w, torch.zeros(4, 96, dtype=torch.bfloat16, device="cuda"))      # k not a multiple of 64
    w = torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(MegakernelError):
        batched.linear(w, torch.zeros(129, 128, dtype=torch.bfloat16, device="cuda"))   # batch above 128
    with pytest.raises(ValueError):
        batched.linear(w, torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda"))


CFG = dict(hidden_size=2048, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
           intermediate_size=8192, vocab_size=4096)


@pytest.mark.parametrize("batch", [16, 5])
def test_two_layer_model_independent_cache_lengths(batch):
    """A 2-layer model, `batch` sequences with different cache lengths, two
    steps.  Oracle: every sequence decoded on its own through the CPU
    interpreter of the batch-1 instruction set (oracle/pyvm.py) on the same
    weights, cache rows and tokens.  Layer 0's appended cache rows must meet
    |a - ref| <= 3e-2 + 1e-2 |ref|; so must everything else, except where two
    layers of 2048-wide fp32 sums in a different order (the tensor core's) put
    single elements just outside the band: there the bound is twice the distance
    of an exactly accumulated restatement from the oracle (helpers.assert_parity),
    as for the batch-1 kernel on wide models."""
    from helpers import assert_parity, build_schedule, exact_matvecs
    from oracle import pyvm
    from thor_megakernels_b200.batched import BatchedDecoder
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig

    max_len = 96
    gpu = LlamaForCausalLM.random_init(LlamaConfig(**CFG), ExtraModelConfig(interleave_rope=True, max_len_override=max_len,
                                                                            max_batch_size=batch), seed=7, device="cuda")
    extra = ExtraModelConfig(interleave_rope=True, max_len_override=max_len)
    cpu = LlamaForCausalLM.random_init(LlamaConfig(**CFG), extra, seed=7, device="cpu")
    exact = LlamaForCausalLM.random_init(LlamaConfig(**CFG), extra, seed=7, device="cpu")
    assert torch.equal(gpu.stacked_params.down_proj.cpu(), cpu.stacked_params.down_proj)
    gen = torch.Generator().manual_seed(3)
    lengths = torch.randint(3, 70, (batch,), generator=gen)
    lengths[0], lengths[-1] = 1, 64   # a sequence with a single cached row, and a block-aligned one
    kv = [torch.randn(gpu.stacked_kv_cache[i].shape, generator=gen).bfloat16() for i in range(2)]
    for i in range(2):
        for b in range(batch):
            kv[i][:, b, int(lengths[b]):] *= 100.0   # garbage beyond every sequence's own length
        gpu.stacked_kv_cache[i].copy_(kv[i].cuda())
    dec = BatchedDecoder(gpu, batch)
    cpu_sched, exact_sched = build_schedule(cpu), build_schedule(exact)
    instr, exact_instr = cpu_sched.get_linear_instructions(), exact_sched.get_linear_instructions()
    tokens = torch.randint(0, CFG["vocab_size"], (batch,), generator=gen).int()
    pos = lengths.int()
    for step in range(2):
        before = [c.clone() for c in gpu.stacked_kv_cache]
        got = dec.step(tokens.cuda(), pos.cuda())
        dec.status()
        want = []
        for b in range(batch):
            p_b = int(pos[b])
            for model in (cpu, exact):
                for i in range(2):
                    model.stacked_kv_cache[i][:, 0] = before[i][:, b].cpu()
            nxt = pyvm.pyvm_step(cpu, cpu_sched, instr, tokens[b].view(1, 1).long(), p_b)
            with exact_matvecs():
                pyvm.pyvm_step(exact, exact_sched, exact_instr, tokens[b].view(1, 1).long(), p_b)
            g, e = cpu_sched.globs, exact_sched.globs
            assert_close(f"layer-0 k row[{b}]", gpu.stacked_kv_cache[0][0, b, p_b], cpu.stacked_kv_cache[0][0, 0, p_b])
            assert_close(f"layer-0 v row[{b}]", gpu.stacked_kv_cache[1][0, b, p_b], cpu.stacked_kv_cache[1][0, 0, p_b])
            assert_parity(f"hidden[{b}]", dec.hidden[b], g.hidden_states, e.hidden_states, layers=2)
            assert_parity(f"k rows[{b}]", gpu.stacked_kv_cache[0][:, b, p_b], cpu.stacked_kv_cache[0][:, 0, p_b],
                          exact.stacked_kv_cache[0][:, 0, p_b], layers=2)
            # the LM head on its own: the oracle's head applied to the residual stream the GPU produced
            head_in = pyvm.rms_norm(dec.hidden[b].cpu(), cpu.lm_head.input_norm.weight, cpu.config.rms_norm_eps)
            assert_close(f"logits[{b}]", dec.logits[b], (cpu.lm_head.lm_head.weight.float() @ head_in.float()).bfloat16())
            assert int(got[b]) == int(dec.logits[b].float().argmax()), "argmax kernel differs from argmax of the logits it read"
            if int(got[b]) != int(nxt):
                ref_logits = cpu.lm_head.lm_head.weight.float() @ pyvm.rms_norm(g.hidden_states, cpu.lm_head.input_norm.weight, cpu.config.rms_norm_eps).float()
                top2 = torch.topk(ref_logits, 2).values
                assert float(top2[0] - top2[1]) <= 0.125
            want.append(int(nxt))
        # rows beyond a sequence's position and other sequences' slots are untouched
        for i in range(2):
            changed = (gpu.stacked_kv_cache[i] != before[i]).any(dim=-1).any(dim=-1)   # [L, B, T]
            for b in range(batch):
                touched = changed[:, b].nonzero()
                assert all(int(t[1]) == int(pos[b]) for t in touched), (b, touched[:4])
        tokens = torch.tensor(want, dtype=torch.int32)
        pos = pos + 1
    dec.close()


def test_out_of_range_tokens_and_positions_are_clamped_and_reported():
    """Token ids and positions live in device memory, so only the device can
    check them: a value outside the vocabulary / the cache is clamped into range
    before anything indexes with it, status() raises, and the step equals the
    step on the clamped values."""
    from thor_megakernels_b200._lib import MegakernelError
    from thor_megakernels_b200.batched import BatchedDecoder
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig

    batch, max_len = 4, 64
    model = LlamaForCausalLM.random_init(LlamaConfig(**CFG), ExtraModelConfig(interleave_rope=True, max_len_override=max_len,
                                                                              max_batch_size=batch), seed=11, device="cuda")
    gen = torch.Generator().manual_seed(5)
    kv = [torch.randn(model.stacked_kv_cache[i].shape, generator=gen).bfloat16().cuda() for i in range(2)]
    dec = BatchedDecoder(model, batch)

    def run(tokens, pos):
        for i in range(2):
            model.stacked_kv_cache[i].copy_(kv[i])
        out = dec.step(torch.tensor(tokens, dtype=torch.int32, device="cuda"), torch.tensor(pos, dtype=torch.int32, device="cuda")).clone()
        return out, dec.logits.clone(), [c.clone() for c in model.stacked_kv_cache]

    bad = run([5, CFG["vocab_size"] + 7, -3, 9], [10, 20, max_len + 100, -1])
    with pytest.raises(MegakernelError):
        dec.status()
    good = run([5, CFG["vocab_size"] - 1, 0, 9], [10, 20, max_len - 1, 0])
    dec.status()   # the error word was cleared, and in-range values leave it clear
    assert torch.equal(bad[0], good[0]) and torch.equal(bad[1], good[1])
    assert all(torch.equal(a, b) for a, b in zip(bad[2], good[2]))
    dec.close()


@pytest.mark.parametrize("rows,k", [(128, 256), (37, 512), (300, 2048)])
def test_native_quantiser_is_bit_exact(rows, k):
    """Codes and scale bytes equal the numpy oracle's (oracle/nvfp4.py); the
    scale bytes sit in the tensor core's 512-byte atoms."""
    import numpy as np

    from oracle import nvfp4 as oracle
    from thor_megakernels_b200 import batched

    torch.manual_seed(rows + k)
    x = torch.randn(rows, k).bfloat16()
    x[0, :32] = 0
    q = batched.quantize_native(x.cuda())
    ts = oracle.tensor_scale_for(x.abs().max().item())
    assert q.tensor_scale == float(ts)
    packed, scales, _ = oracle.quantize(x.float().numpy(), ts)
    assert np.array_equal(q.packed.cpu().numpy(), packed)
    assert np.array_equal(q.canonical_scales().cpu().numpy(), scales)
    # rows of the last atom beyond `rows` keep scale 0
    native = q.scales.cpu().numpy().reshape(-1, k // 64, 32, 4, 4)
    r = rows  # first row that does not exist
    if r % 128:
        assert native[r // 128, :, r % 32, (r % 128) // 32, :].sum() == 0


@pytest.mark.parametrize("n,k", [(128, 256), (256, 1024), (3072, 2048), (2048, 8192), (1000, 2048)])
@pytest.mark.parametrize("batch", [16, 64, 128, 37])
def test_block_scaled_nvfp4_linear(n, k, batch):
    """tcgen05 block-scaled NVFP4 linear against the oracle: both operands
    decoded with the numpy oracle's decoder, exact (float64) dot products, one
    bf16 rounding.  Tolerance: relative L2 <= 1e-3 (the reference's gate,
    tools/analysis/nvfp4/check.py:43) and the element band."""
    import numpy as np

    from oracle import nvfp4 as oracle
    from thor_megakernels_b200 import batched

    gen = torch.Generator(device="cuda").manual_seed(n + k + batch)
    w = (torch.randn(n, k, device="cuda", generator=gen) * 0.02).bfloat16()
    x = torch.randn(batch, k, device="cuda", generator=gen).bfloat16()
    qw, qx = batched.quantize_native(w), batched.quantize_native(x)
    got = batched.linear_nvfp4(qw, qx)
    batched.check_errors()
    dw = oracle.dequantize(qw.packed.cpu().numpy(), qw.canonical_scales().cpu().numpy(), qw.tensor_scale).astype(np.float64)
    dx = oracle.dequantize(qx.packed.cpu().numpy(), qx.canonical_scales().cpu().numpy(), qx.tensor_scale).astype(np.float64)
    want = torch.from_numpy(dx @ dw.T).float().bfloat16().float()
    assert got.shape == (batch, n)
    assert rel_l2(got.float().cpu(), want) <= 1e-3
    assert_close("nvfp4 linear", got, want)


def test_two_layer_model_nvfp4_weights_and_activations():
    """The batched step with NVFP4 weights: every linear is the block-scaled
    tensor-core MMA on activations quantised on the fly.  Oracle:
    oracle/nvfp4_w4a4.py per sequence, decoding exactly the weight bytes the
    device quantiser produced.  Quantising activations turns a single-ulp bf16
    difference at a rounding boundary into a different 4-bit code, so beyond the
    first linear the comparison is statistical: layer 0's appended K row (which
    only depends on the embedding and one linear) must meet the band; hidden
    state and logits must stay within 3 % NRMSE of the oracle, the level at which
    two exact implementations with different summation order already differ."""
    import numpy as np

    from oracle import nvfp4 as fmt, nvfp4_model, nvfp4_w4a4
    from thor_megakernels_b200.batched import BatchedDecoder
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig
    from thor_megakernels_b200.nvfp4 import quantize_model

    batch, max_len = 16, 96
    gpu = LlamaForCausalLM.random_init(LlamaConfig(**CFG), ExtraModelConfig(interleave_rope=True, max_len_override=max_len,
                                                                            max_batch_size=batch), seed=7, device="cuda")
    cpu = LlamaForCausalLM.random_init(LlamaConfig(**CFG), ExtraModelConfig(interleave_rope=True, max_len_override=max_len,
                                                                            max_batch_size=batch), seed=7, device="cpu")
    q = quantize_model(gpu)

    def to_oracle(w):
        dq = fmt.dequantize(w.packed.cpu().numpy(), w.scales.cpu().numpy(), w.tensor_scale)
        return nvfp4_model.QuantMatrix(None, None, np.float32(w.tensor_scale), torch.from_numpy(dq))

    layers = [nvfp4_model.QuantLayer(*(to_oracle(q[k][i]) for k in ("qkv", "o", "up", "gate", "down"))) for i in range(2)]
    head = to_oracle(q["lm_head"])
    gen = torch.Generator().manual_seed(3)
    lengths = torch.randint(3, 70, (batch,), generator=gen)
    for i in range(2):
        kv = torch.randn(gpu.stacked_kv_cache[i].shape, generator=gen).bfloat16()
        for b in range(batch):
            kv[:, b, int(lengths[b]):] *= 100.0
        gpu.stacked_kv_cache[i].copy_(kv.cuda())
        cpu.stacked_kv_cache[i].copy_(kv)
    dec = BatchedDecoder(gpu, batch, quantized=q)
    tokens = torch.randint(0, CFG["vocab_size"], (batch,), generator=gen).int()
    got = dec.step(tokens.cuda(), lengths.int().cuda())
    dec.status()
    emb = cpu.model.embed_tokens.embed_tokens.weight
    worst_h, worst_l = 0.0, 0.0
    for b in range(batch):
        hidden, logits, _ = nvfp4_w4a4.decode_step(cpu, layers, head, emb[int(tokens[b])], int(lengths[b]), cache_slot=b)
        assert_close(f"layer-0 k row[{b}]", gpu.stacked_kv_cache[0][0, b, int(lengths[b])], cpu.stacked_kv_cache[0][0, b, int(lengths[b])])
        worst_h = max(worst_h, nrmse(dec.hidden[b], hidden))
        worst_l = max(worst_l, nrmse(dec.logits[b], logits))
        assert int(got[b]) == int(dec.logits[b].float().argmax())
    print(f"worst NRMSE over {batch} sequences: hidden {worst_h:.4f}, logits {worst_l:.4f}")
    assert worst_h <= 0.03 and worst_l <= 0.03
    dec.close()


@pytest.mark.parametrize("batch", [1, 16])
def test_fp4_chain_of_dependent_linears(batch):
    """``mk_fp4_chain_*`` (the counterpart of the reference's vm_prepare / vm_run,
    experimental/native_fp4_vm/vm.cu:14-63): up projection 2048 -> 8192 whose
    output feeds a down projection 8192 -> 2048, inputs quantised on the fly.
    Oracle per operand: numpy quantiser on the operand's actual input, decoded
    operands, float64 dot products, one bf16 rounding."""
    import numpy as np

    from oracle import nvfp4 as oracle
    from thor_megakernels_b200 import batched

    gen = torch.Generator(device="cuda").manual_seed(40 + batch)
    w1 = (torch.randn(8192, 2048, device="cuda", generator=gen) * 0.02).bfloat16()
    w2 = (torch.randn(2048, 8192, device="cuda", generator=gen) * 0.02).bfloat16()
    x = torch.randn(batch, 2048, device="cuda", generator=gen).bfloat16()
    y1 = torch.zeros(batch, 8192, dtype=torch.bfloat16, device="cuda")
    y2 = torch.zeros(batch, 2048, dtype=torch.bfloat16, device="cuda")
    q1, q2 = batched.quantize_native(w1), batched.quantize_native(w2)
    scales = [float(oracle.tensor_scale_for(x.abs().max().item())), 0.9 / (6 * 448)]
    chain = batched.Fp4Chain([q1, q2], [x, y1], [y1, y2], scales)
    for _ in range(2):   # a second run reuses the scratch
        chain.run()
    chain.status()

    def expect(qw, inp, ts):
        dw = oracle.dequantize(qw.packed.cpu().numpy(), qw.canonical_scales().cpu().numpy(), qw.tensor_scale).astype(np.float64)
        _, _, dx = oracle.quantize(inp.float().cpu().numpy(), np.float32(ts))
        return torch.from_numpy(dx.astype(np.float64) @ dw.T).float().bfloat16().float()

    want1 = expect(q1, x, scales[0])
    assert rel_l2(y1.float().cpu(), want1) <= 1e-3
    assert_close("chain operand 0", y1, want1)
    want2 = expect(q2, y1, scales[1])     # from the GPU's own y1: the second quantiser sees exactly these values
    assert rel_l2(y2.float().cpu(), want2) <= 1e-3
    assert_close("chain operand 1", y2, want2)
    chain.close()


def test_fp4_chain_refuses_unaligned_operands():
    import ctypes as C

    from thor_megakernels_b200 import _lib

    lib = _lib.load()
    op = (_lib.MkFp4ChainOperand * 1)()
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    for f in ("input", "output", "w_packed", "w_scales_native"):
        setattr(op[0], f, buf.data_ptr())
    op[0].m, op[0].k, op[0].input_tensor_scale, op[0].alpha = 128, 192, 1.0, 1.0   # k not a multiple of 256
    handle = C.c_void_p()
    assert lib.mk_fp4_chain_prepare(op, 1, 1, 1, C.byref(handle)) == _lib.MK_ERR_BAD_ARGUMENT
    op[0].k, op[0].input_tensor_scale = 256, 0.0
    assert lib.mk_fp4_chain_prepare(op, 1, 1, 1, C.byref(handle)) == _lib.MK_ERR_BAD_ARGUMENT
