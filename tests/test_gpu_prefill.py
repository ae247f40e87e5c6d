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
    # greedy token: the reference's choice, or one its own logits rank within rounding noise of the best
    logits = ref.lm_head.lm_head(ref.lm_head.input_norm(out.hidden_states[0, -1])).float()
    assert float(logits[int(tok)]) >= float(logits.max()) - (3e-2 + 1e-2 * float(logits.max().abs())), (int(tok), int(logits.argmax()))
    assert nrmse(dec.logits[0], logits) <= 2e-2
    dec.close()


def test_decode_continues_from_a_device_prefill():
    """Prompt on the device, then one batch-1 megakernel step from that cache: the same logits (within rounding
    noise) as after the PyTorch prefill, and the same cache row appended."""
    from helpers import build_schedule
    from thor_megakernels_b200.generators import MK_FusedGenerator
    from thor_megakernels_b200.model_types import BatchState
    from thor_megakernels_b200.runtime import MK_STEP_EMBED, MK_STEP_RESET_BARRIERS

    n = 45
    prompt = torch.randint(0, CFG["vocab_size"], (n,), generator=torch.Generator().manual_seed(2))
    token = torch.tensor([1234], dtype=torch.int32, device="cuda")
    results = []
    for device_prefill in (False, True):
        model = build("cuda", 128)
        sched = build_schedule(model, "b200")
        gen = MK_FusedGenerator(model, sched)
        if device_prefill:
            gen.prefill(prompt.cuda())
        else:
            model(BatchState(input_ids=prompt.cuda()[None], position_ids=torch.arange(n, device="cuda")[None]))
        gen.mk.step(n, flags=MK_STEP_EMBED | MK_STEP_RESET_BARRIERS, token_in=token)
        torch.cuda.synchronize()
        gen.mk.status()
        results.append((sched.globs.logits.clone(), model.stacked_kv_cache[0][:, 0, n].clone(), model.stacked_kv_cache[1][:, 0, n].clone()))
    (la, ka, va), (lb, kb, vb) = results
    assert nrmse(lb, la) <= 1e-2, nrmse(lb, la)
    assert_close("layer-0 k row of the decode step", kb[0], ka[0])
    assert nrmse(kb[1], ka[1]) <= 1e-2 and nrmse(vb[1], va[1]) <= 1e-2
