"""Runs a few decode steps of the benchmark model and nothing else, so that a
profiler sees only megakernel launches:

    ncu --set full --clock-control none -k regex:decode_step -s 3 -c 1 \\
        python -m thor_megakernels_b200.profile_step --steps 4

Same model, schedule and cache contents as ``bench.py`` (Llama-3.2-1B
architecture, bf16, 16-token context); ``--layers`` shrinks the model for a
smaller capture.  Prints the mean step time measured with CUDA events.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def main():
    import torch

    import bench
    from thor_megakernels_b200.runtime import (MK_STEP_EMBED, MK_STEP_RESET_BARRIERS, MK_STEP_WRITE_TOKEN, Megakernel)

    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--pos", type=int, default=60)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--arch", default="1b", choices=["1b", "8b"], help="8b: Llama-3.1-8B layer shapes, --pos cached positions")
    ap.add_argument("--partitions", type=int, default=18, help="attention slices per KV head (8b only)")
    ap.add_argument("--nvfp4", action="store_true", help="NVFP4 weight-only linears instead of bf16 weights")
    args = ap.parse_args()
    if args.arch == "8b":
        # Llama-3.1-8B layer shapes with a long cache (attention split into slices), few layers to keep the capture small
        from thor_megakernels_b200.demos.latency.scheduler import LatencyScheduleBuilder
        from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
        from thor_megakernels_b200.model_types import ExtraModelConfig
        from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

        cfg = dict(bench.MODEL_8B, num_hidden_layers=args.layers or 4)
        device = torch.device("cuda:0")
        extra = ExtraModelConfig(interleave_rope=True, max_len_override=args.pos + 16)
        model = LlamaForCausalLM.random_init(LlamaConfig(**cfg), extra, seed=4, device=device, generate_on=device)
        gen = torch.Generator(device=device).manual_seed(3)
        for cache in model.stacked_kv_cache:
            cache[:, :, :args.pos] = torch.randn(cache[:, :, :args.pos].shape, generator=gen, device=device).bfloat16()
        sched = LatencyScheduleBuilder.build(model, skip_attn_reduction=args.partitions == 1,
                                             num_attention_partitions=args.partitions)
        tensorize_instructions(sched.globs, assign_to_sms("rr", schedule=sched))
        sched.globs.barriers.zero_()
    else:
        if args.layers is not None:
            bench.MODEL.update(num_hidden_layers=args.layers)
        model, sched = bench.build_gpu_model(torch.device("cuda:0"))
    quantized = None
    if args.nvfp4:
        from thor_megakernels_b200.nvfp4 import quantize_model

        quantized = quantize_model(model)
    mk = Megakernel.from_globals(sched.globs, embed_w=model.model.embed_tokens.embed_tokens.weight.data, quantized=quantized)
    tok = torch.tensor([17], dtype=torch.int32, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    flags = MK_STEP_EMBED | MK_STEP_RESET_BARRIERS | MK_STEP_WRITE_TOKEN
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    mk.step(args.pos, flags=flags, token_in=tok, token_out=out)
    torch.cuda.synchronize()
    start.record()
    for _ in range(args.steps):
        mk.step(args.pos, flags=flags, token_in=tok, token_out=out)
    end.record()
    torch.cuda.synchronize()
    mk.status()
    print(f"{args.steps} steps at position {args.pos}: {start.elapsed_time(end) / args.steps:.4f} ms/step, token {int(out)}")


if __name__ == "__main__":
    main()
