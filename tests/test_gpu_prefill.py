"""Prompt processing on the device (``mk_prefill_batched``) against the plain
PyTorch forward the reference uses for prefill (megakernels/scripts/generate.py:
125-132; restated in ``thor_megakernels_b200/llama.py``), run on the CPU with
the same seeded weights.  Tolerance: layer-0 cache rows within the stated band
``|a - ref| <= 3e-2 + 1e-2 |ref|``; deeper rows and the last hidden state by
relative error (bf16 linears accumulate differently on the two devices); the
greedy token after the prompt must match."""
import pytest
import torch

from helpers import assert_close, nrmse

pytestmark = pytest.mark.gpu

CFG = dict(hidden_size=2048, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
           intermediate_size=8192, vocab_size=4096)


def build(device, max_len):
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig

    return LlamaForCausalLM.random_init(LlamaConfig(**CFG), ExtraModelConfig(interleave_rope=True, max_len_override=max_len),
                                        seed=21, device=device)


@pytest.mark.parametrize("n", [1, 37, 128, 200])
def test_prefill_fills_the_cache_and_picks_the_same_token(n):
    from thor_megakernels_b200.batched import BatchedDecoder
    from thor_megakernels_b200.model_types import BatchState

    ref, model = build("cpu", 256), build("cuda", 256)
    prompt = torch.randint(0, CFG["vocab_size"], (n,), generator=torch.Generator().manual_seed(n))
    out = ref(BatchState(input_ids=prompt[None], position_ids=torch.arange(n)[None]))
    dec = BatchedDecoder(model, max_batch=128)
    tok = dec.prefill(prompt.to("cuda", torch.int32))
    dec.status()
    for i, name in enumerate(("k", "v")):
        got, want = model.stacked_kv_cache[i][:, 0, :n], ref.stacked_kv_cache[i][:, 0, :n]
        assert_close(f"layer-0 {name} rows", got[0], want[0])
        assert nrmse(got[1], want[1]) <= 1e-2, (name, nrmse(got[1], want[1]))
        assert not bool(model.stacked_kv_cache[i][:, 0, n:].any())   # nothing written beyond the prompt
    assert int(tok) == int(out.output_ids[0, -1])
    dec.close()


def test_decode_continues_from_a_device_prefill():
    """Prompt on the device, then the batch-1 megakernel decodes from that cache: same tokens as after a PyTorch prefill."""
    from helpers import build_schedule
    from thor_megakernels_b200.generators import MK_FusedGenerator
    from thor_megakernels_b200.model_types import BatchState

    n, ntok = 45, 6
    prompt = torch.randint(0, CFG["vocab_size"], (n,), generator=torch.Generator().manual_seed(2))
    streams = []
    for device_prefill in (False, True):
        model = build("cuda", 128)
        gen = MK_FusedGenerator(model, build_schedule(model, "b200"))
        out_tokens = torch.zeros(1, ntok, dtype=torch.long, device="cuda")
        if device_prefill:
            out_tokens[0, 0] = gen.prefill(prompt.cuda())[0]
        else:
            out = model(BatchState(input_ids=prompt.cuda()[None], position_ids=torch.arange(n, device="cuda")[None]))
            out_tokens[0, 0] = out.output_ids[0, -1]
        gen.generate(out_tokens, n, ntok - 1)
        torch.cuda.synchronize()
        gen.mk.status()
        streams.append(out_tokens[0].tolist())
    assert streams[0] == streams[1]
