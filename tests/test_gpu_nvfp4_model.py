"""NVFP4 weight-only decode through the megakernel against the CPU oracle that
follows the reference's quantised-model rules (oracle/nvfp4_model.py):
weights quantised on the device (bit-exact with the oracle quantiser, checked in
test_gpu_nvfp4.py), bf16 activations and KV cache."""
import numpy as np
import pytest
import torch

from helpers import assert_close, build_model, build_schedule

pytestmark = pytest.mark.gpu

CFG = dict(hidden_size=2048, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
           intermediate_size=8192, vocab_size=4096)


def test_two_layer_model_three_steps():
    from oracle import nvfp4 as fmt, nvfp4_model
    from thor_megakernels_b200.nvfp4 import quantize_model
    from thor_megakernels_b200.runtime import (MK_STEP_EMBED, MK_STEP_RESET_BARRIERS, MK_STEP_WRITE_TOKEN, Megakernel)

    cpu = build_model(CFG, 64, device="cpu", seed=5)
    gpu = build_model(CFG, 64, device="cuda", seed=5)
    q = quantize_model(gpu)

    # the oracle decodes exactly the bytes the device produced
    def to_oracle(w):
        dq = fmt.dequantize(w.packed.cpu().numpy(), w.scales.cpu().numpy(), w.tensor_scale)
        return nvfp4_model.QuantMatrix(None, None, np.float32(w.tensor_scale), torch.from_numpy(dq))

    layers = [nvfp4_model.QuantLayer(*(to_oracle(q[k][i]) for k in ("qkv", "o", "up", "gate", "down")))
              for i in range(CFG["num_hidden_layers"])]
    head = to_oracle(q["lm_head"])

    gen = torch.Generator().manual_seed(9)
    ctx = 12
    for idx in range(2):
        kv = torch.randn(cpu.stacked_kv_cache[idx][:, :, :ctx].shape, generator=gen).bfloat16()
        cpu.stacked_kv_cache[idx][:, :, :ctx] = kv
        gpu.stacked_kv_cache[idx][:, :, :ctx] = kv.cuda()

    sched = build_schedule(gpu)
    g = sched.globs
    emb = gpu.model.embed_tokens.embed_tokens.weight.data
    mk = Megakernel.from_globals(g, embed_w=emb, quantized=q)
    tok_in = torch.tensor([77], dtype=torch.int32, device="cuda")
    tok_out = torch.zeros(1, dtype=torch.int32, device="cuda")
    g.barriers.zero_()
    token = 77
    for step in range(3):
        pos = ctx + step
        hidden, logits, last = nvfp4_model.decode_step(cpu, layers, head, cpu.model.embed_tokens.embed_tokens.weight[token], pos)
        tok_in.fill_(token)
        mk.step(pos, flags=MK_STEP_EMBED | MK_STEP_RESET_BARRIERS | MK_STEP_WRITE_TOKEN, token_in=tok_in, token_out=tok_out)
        mk.status()
        assert_close("silu_out", g.silu_out, last["silu_out"])
        assert_close("attn_out", g.attn_out, last["attn_out"])
        assert_close("hidden", g.hidden_states, hidden)
        assert_close("logits", g.logits, logits)
        assert_close("k row", gpu.stacked_kv_cache[0][:, 0, pos], cpu.stacked_kv_cache[0][:, 0, pos])
        want = int(logits.float().argmax())
        if int(tok_out) != want:
            top2 = torch.topk(logits.float(), 2).values
            assert float(top2[0] - top2[1]) <= 0.125
        token = want
