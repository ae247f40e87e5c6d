"""Checkpoint loading with tensor-parallel slicing, on a synthetic safetensors
checkpoint written by this repository (reference megakernels/utils.py:22-97,
llama.py:583-711)."""
import json

import pytest
import torch

from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
from thor_megakernels_b200.model_types import ExtraModelConfig
from thor_megakernels_b200.utils import compute_shard_bounds, load_safetensors_repo

CFG = dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=32,
           intermediate_size=512, vocab_size=320, tie_word_embeddings=False)


def write_checkpoint(tmp_path, sharded: bool):
    from safetensors.torch import save_file

    raw = LlamaForCausalLM.random_init(LlamaConfig(**CFG), ExtraModelConfig(interleave_rope=True, max_len_override=32), seed=11,
                                       finalize=False)
    state = raw.to_hf_state_dict()
    cfg_json = dict(CFG, rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=131072,
                    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                      original_max_position_embeddings=8192))
    (tmp_path / "config.json").write_text(json.dumps(cfg_json))
    if not sharded:
        save_file(state, str(tmp_path / "model.safetensors"))
    else:
        names = sorted(state)
        halves = {"model-00001-of-00002.safetensors": names[::2], "model-00002-of-00002.safetensors": names[1::2]}
        weight_map = {}
        for fname, keys in halves.items():
            save_file({k: state[k] for k in keys}, str(tmp_path / fname))
            weight_map.update({k: fname for k in keys})
        (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    raw.finalize()
    return raw


def test_shard_bounds_spread_the_remainder_over_the_first_shards():
    assert [compute_shard_bounds([10], 0, 3, i) for i in range(3)] == [slice(0, 4), slice(4, 7), slice(7, 10)]
    assert compute_shard_bounds([4, 8], 1, 2, 1) == slice(4, 8)


@pytest.mark.parametrize("sharded", [False, True])
def test_whole_model_round_trip(tmp_path, sharded):
    want = write_checkpoint(tmp_path, sharded)
    got = LlamaForCausalLM.from_pretrained(tmp_path, ExtraModelConfig(interleave_rope=True, max_len_override=32))
    for name in ("qkv_proj", "o_proj", "up_proj", "gate_proj", "down_proj", "attn_ln_weight", "mlp_ln_weight"):
        assert torch.equal(getattr(got.stacked_params, name), getattr(want.stacked_params, name)), name
    assert torch.equal(got.lm_head.lm_head.weight, want.lm_head.lm_head.weight)
    assert torch.equal(got.model.embed_tokens.embed_tokens.weight, want.model.embed_tokens.embed_tokens.weight)
    assert torch.equal(got.model.rope_cos, want.model.rope_cos)
    assert got.stacked_kv_cache[0].shape == want.stacked_kv_cache[0].shape


@pytest.mark.parametrize("world", [2])
def test_tensor_parallel_load_equals_sharding_the_whole_model(tmp_path, world):
    """A rank that loads with tp_size > 1 reads only its slices and ends up with
    exactly the weights ``tp.shard_model`` cuts out of the whole model."""
    from thor_megakernels_b200.tp import shard_model

    whole = write_checkpoint(tmp_path, sharded=True)
    for rank in range(world):
        extra = ExtraModelConfig(interleave_rope=True, max_len_override=32, tp_size=world, tp_rank=rank)
        got = LlamaForCausalLM.from_pretrained(tmp_path, extra)
        want = shard_model(whole, rank, world)
        assert got.config.num_attention_heads == want.config.num_attention_heads
        assert got.config.intermediate_size == want.config.intermediate_size
        for name in ("qkv_proj", "o_proj", "up_proj", "gate_proj", "down_proj"):
            assert torch.equal(getattr(got.stacked_params, name), getattr(want.stacked_params, name)), (rank, name)
        assert got.stacked_kv_cache[0].shape == want.stacked_kv_cache[0].shape


def test_missing_checkpoint_and_unsplittable_shapes(tmp_path):
    with pytest.raises(FileNotFoundError):
        load_safetensors_repo(tmp_path, {"x"}, "cpu")
    write_checkpoint(tmp_path, sharded=False)
    with pytest.raises(ValueError):
        LlamaForCausalLM.from_pretrained(tmp_path, ExtraModelConfig(tp_size=3, tp_rank=0, max_len_override=32))
