"""Tensor-parallel decode over the GPUs of one node, one process per GPU.

The shard layout is the reference model's (``megakernels/llama.py``): query and
KV heads divided by the number of ranks (:192-207), so q/k/v rows are split by
head; o_proj and down_proj by input columns, up/gate by output rows
(:308-310, :665-691); here the LM head is also split by vocabulary rows and the
embedding stays whole.  Norm weights and rotary tables are replicated.

The reference runs that layout only through PyTorch with NCCL collectives
between blocks.  Here every rank runs the decode megakernel on its shard and
the two all-reduces per layer happen inside the kernel over NVLink peer memory
(``mk_tp_init`` / ``mk_tp_connect`` in ``include/b200_megakernel.h``);
``torch.distributed`` is used once, to all-gather the 64-byte IPC handles.
"""
from __future__ import annotations

import dataclasses
from types import SimpleNamespace

import torch

from .llama import LlamaConfig, StackedParams


def check_divisible(cfg: LlamaConfig, world: int):
    if cfg.num_key_value_heads % world or cfg.num_attention_heads % world:
        raise ValueError(f"{cfg.num_attention_heads} query / {cfg.num_key_value_heads} KV heads do not divide over {world} ranks")
    if cfg.intermediate_size % (256 * world):
        raise ValueError(f"intermediate_size {cfg.intermediate_size}: every rank needs a multiple of 256 columns")
    if cfg.vocab_size % (16 * world):
        raise ValueError(f"vocab_size {cfg.vocab_size}: every rank needs a multiple of 16 rows")


def shard_config(cfg: LlamaConfig, world: int) -> LlamaConfig:
    """The configuration one rank's kernel sees: its share of heads, FFN columns
    and vocabulary; hidden size and layer count unchanged."""
    check_divisible(cfg, world)
    return dataclasses.replace(
        cfg,
        num_attention_heads=cfg.num_attention_heads // world,
        num_key_value_heads=cfg.num_key_value_heads // world,
        intermediate_size=cfg.intermediate_size // world,
        vocab_size=cfg.vocab_size // world,
        tie_word_embeddings=False,
    )


def shard_slices(cfg: LlamaConfig, rank: int, world: int) -> dict:
    """Row / column ranges of rank ``rank`` in the whole model's stacked tensors."""
    check_divisible(cfg, world)
    d = cfg.head_dim
    hq, hkv = cfg.num_attention_heads // world, cfg.num_key_value_heads // world
    inter, vocab = cfg.intermediate_size // world, cfg.vocab_size // world
    q0 = rank * hq * d
    k0 = cfg.num_attention_heads * d + rank * hkv * d
    v0 = (cfg.num_attention_heads + cfg.num_key_value_heads) * d + rank * hkv * d
    return dict(
        q_rows=(q0, q0 + hq * d), k_rows=(k0, k0 + hkv * d), v_rows=(v0, v0 + hkv * d),
        o_cols=(q0, q0 + hq * d),
        ffn=(rank * inter, (rank + 1) * inter),
        vocab=(rank * vocab, (rank + 1) * vocab),
        kv_heads=(rank * hkv, (rank + 1) * hkv),
    )


def shard_model(model, rank: int, world: int):
    """Rank ``rank``'s share of a finalised model container, as an object with the
    attributes the schedule builder and the kernel handle read (``config``,
    ``stacked_params``, ``stacked_kv_cache``, ``lm_head``, ``model.rope_*``,
    ``model.embed_tokens``).  Weights are copied into contiguous tensors; the KV
    cache keeps the rank's heads of whatever the whole model's cache holds."""
    cfg = model.config
    sl = shard_slices(cfg, rank, world)
    sp = model.stacked_params
    (q0, q1), (k0, k1), (v0, v1) = sl["q_rows"], sl["k_rows"], sl["v_rows"]
    (o0, o1), (f0, f1), (t0, t1), (h0, h1) = sl["o_cols"], sl["ffn"], sl["vocab"], sl["kv_heads"]
    stacked = StackedParams(
        qkv_proj=torch.cat([sp.qkv_proj[:, q0:q1], sp.qkv_proj[:, k0:k1], sp.qkv_proj[:, v0:v1]], dim=1).contiguous(),
        o_proj=sp.o_proj[:, :, o0:o1].contiguous(),
        attn_ln_weight=sp.attn_ln_weight,
        mlp_ln_weight=sp.mlp_ln_weight,
        up_proj=sp.up_proj[:, f0:f1].contiguous(),
        gate_proj=sp.gate_proj[:, f0:f1].contiguous(),
        down_proj=sp.down_proj[:, :, f0:f1].contiguous(),
    )
    k, v = model.stacked_kv_cache
    cache = (k[:, :, :, h0:h1].contiguous(), v[:, :, :, h0:h1].contiguous())
    head_w = model.lm_head.lm_head.weight.data[t0:t1].contiguous()
    return SimpleNamespace(
        config=shard_config(cfg, world),
        extra_config=model.extra_config,
        device=model.device,
        dtype=model.dtype,
        stacked_params=stacked,
        stacked_kv_cache=cache,
        lm_head=SimpleNamespace(input_norm=SimpleNamespace(weight=model.lm_head.input_norm.weight),
                                lm_head=SimpleNamespace(weight=head_w)),
        model=SimpleNamespace(rope_cos=model.model.rope_cos, rope_sin=model.model.rope_sin,
                              embed_tokens=model.model.embed_tokens),
        tp_rank=rank,
        tp_world=world,
        vocab_offset=t0,
    )


class TensorParallelDecoder:
    """Greedy decode of one sequence with the model split over ``world`` GPUs.

    Every rank constructs this with the same whole model (same seed), its own
    ``rank`` and an initialised ``torch.distributed`` process group; the whole
    model can be dropped afterwards.  ``decode`` must be called by all ranks with
    the same arguments and returns the same tokens on every rank."""

    def __init__(self, model, rank: int, world: int, schedule: str = "auto", group=None,
                 num_attention_partitions: int = 1, nvfp4_weights: bool = False):
        import torch.distributed as dist

        from .demos.latency.scheduler import LatencyScheduleBuilder
        from .runtime import Megakernel
        from .scheduler import assign_to_sms, tensorize_instructions

        self.rank, self.world = rank, world
        self.local = shard_model(model, rank, world)
        split = num_attention_partitions > 1
        if schedule == "auto":  # the layout measured fastest for the weight format
            schedule = "rr" if nvfp4_weights else "b200"
        together = schedule == "b200"  # one SM owns all column slices of its down-projection rows
        self.schedule = LatencyScheduleBuilder.build(self.local, skip_attn_reduction=not split,
                                                     num_attention_partitions=num_attention_partitions,
                                                     down_rows_together=together)
        tensorize_instructions(self.schedule.globs, assign_to_sms("rrk" if together else schedule, schedule=self.schedule))
        quantized = None
        if nvfp4_weights:  # every rank quantises its own shard (block scales run along K, which only o/down split)
            from .nvfp4 import quantize_model

            quantized = quantize_model(self.local)
        self.mk = Megakernel.from_globals(self.schedule.globs,
                                          embed_w=model.model.embed_tokens.embed_tokens.weight.data,
                                          quantized=quantized)
        self.schedule.globs.barriers.zero_()
        mine = self.mk.tp_init(rank, world, self.local.vocab_offset)
        handles: list = [None] * world
        dist.all_gather_object(handles, mine, group=group)
        self.mk.tp_connect(handles)
        torch.cuda.synchronize(self.local.device)
        dist.barrier(group=group)  # nobody launches before every rank has mapped its peers

    def decode(self, first_token: int | torch.Tensor, count: int, start_pos: int) -> torch.Tensor:
        dev = self.local.device
        if not isinstance(first_token, torch.Tensor):
            first_token = torch.tensor([int(first_token)], dtype=torch.int32, device=dev)
        out = torch.empty(count, dtype=torch.int32, device=dev)
        self.mk.decode(first_token.to(torch.int32), out, start_pos, count)
        return out

    def logits(self) -> torch.Tensor:
        """This rank's slice of the last step's logits (vocabulary rows
        ``vocab_offset`` .. ``vocab_offset + vocab/world``)."""
        return self.schedule.globs.logits

    def close(self):
        self.mk.close()
