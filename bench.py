"""Decode benchmark: Llama-3.2-1B architecture, bf16, batch 1, greedy.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One *step* is one request of the headline workload: a 16-token context already
in the KV cache and 100 greedy decode tokens at positions 16..115 (seeded
synthetic weights N(0, 0.02), synthetic prompt/KV).  The JSON line reports

* ``value``      tokens/s with everything resident on the device: 100 launches of
                 the megakernel per request, token fed back on the device;
* ``e2e``        the same metric through ``Generator.generate`` with host
                 buffers: the first token comes from pinned host memory and the
                 100 produced tokens are read back, every request;
* ``roofline``   algorithmic bytes per launch (linear weights + KV read + KV
                 written) over the mean launch duration, against the measured
                 HBM copy bandwidth;
* ``cpu_baseline`` the CPU oracle (a port of the reference's PyTorch
                 interpreter) timed on this box's cores over a few tokens.

``--impl reference`` times only that CPU interpreter (one token per step).

With N > 1 (under torchrun) the SAME request is decoded with the model split
over the N GPUs (tensor parallel: heads, FFN columns and vocabulary sharded,
the two all-reduces per layer inside the kernel over NVLink peer memory;
``"scaling": "strong"``).  Before timing, a 2-layer model is decoded both split
and whole and the agreement goes into ``tp_parity``.  At every N the line also
carries ``llama8b_tp``: the Llama-3.1-8B architecture at batch 1 with 8192
cached positions on the same N GPUs, bf16 and NVFP4 weight-only.

Other workloads: ``--workload llama1b-batched`` decodes 16 / 64 / 128 sequences
with independent cache lengths per step (tcgen05 linears); ``llama8b-tp`` /
``llama1b-tp`` run only the split decode; ``gemv`` the single-operator GEMV (bf16 and NVFP4 weights, batch 1 and
4); ``llama1b-nvfp4-4k`` the NVFP4 weight-only megakernel against bf16 weights
at 4096 cached positions; ``timeline`` one step with per-instruction clock
stamps, summarised per opcode; ``profile-step`` a few bare steps for a profiler
(``--arch 8b --layers 4 --pos 8192`` for the 8B shapes).  ``--schedule`` picks
the queue assignment policy (rr, zz, wave, dag).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

PROMPT_LEN = 16
TOKENS_PER_REQUEST = 100
# the headline request; both arms (this library and --impl reference) and every N name it the same way
HEADLINE_WORKLOAD = "llama-3.2-1b-arch bf16 batch-1 greedy decode: 16-token context, 100 tokens (pos 16..115)"
FALLBACK_HBM_GBS = 6650.0  # used only when MEASURED_PEAKS.json is absent

MODEL = dict(hidden_size=2048, num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
             intermediate_size=8192, vocab_size=128256)


MODEL_8B = dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=14336, vocab_size=128256, tie_word_embeddings=False,
                rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192))
TP_WORKLOADS = {
    # name: (model, cached positions, tokens per step, seed)
    "llama8b-tp": (MODEL_8B, 8192, 64, 4),
    "llama1b-tp": (MODEL, PROMPT_LEN, TOKENS_PER_REQUEST, 0),
}


def linear_weight_bytes(cfg: dict) -> int:
    h, inter, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * d
    per_layer = (qkv + h + 2 * inter) * h + h * inter
    return 2 * (cfg["num_hidden_layers"] * per_layer + cfg["vocab_size"] * h)


def kv_bytes_per_position(cfg: dict) -> int:
    return 2 * 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"]


def algorithmic_bytes_per_request(cfg: dict) -> int:
    """Sum over the 100 launches of: every linear weight once, the cached K/V of
    positions 0..pos, and the appended K/V row."""
    kv = kv_bytes_per_position(cfg)
    total = 0
    for pos in range(PROMPT_LEN, PROMPT_LEN + TOKENS_PER_REQUEST):
        total += linear_weight_bytes(cfg) + kv * (pos + 1) + kv
    return total


def measured_hbm_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (no MEASURED_PEAKS.json)"


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, sm_max, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [x for x in sm if x > 0]
        return {"sm_mhz": statistics.median(busy or sm), "sm_max_mhz": max(sm_max), "reasons": sorted(reasons),
                "samples": len(sm)}


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        backend = "nccl" if torch.cuda.is_available() else "gloo"
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
        # NCCL prints its version banner on standard output when the first communicator is created; this
        # script's standard output carries one JSON line and nothing else, so the banner goes to stderr.
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group(backend=backend)
            dist.barrier()
            if torch.cuda.is_available():
                torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    return rank, world, local


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda" if torch.cuda.is_available() else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def pick_schedule(requested: str, weights: str = "bf16") -> str:
    """``auto``: the layout measured fastest for the weight format - ``b200`` for bf16,
    the reference's round robin for NVFP4 weight-only (its consumer is bound by decoding,
    not by hand-offs, and runs one slice per instruction faster)."""
    if requested != "auto":
        return requested
    return "rr" if weights == "nvfp4" else "b200"


def make_schedule(model, schedule: str, **kwargs):
    """``b200``: the library's own layout (one SM owns all column slices of its
    down-projection rows); rr / zz / wave / dag: the reference's layout under
    that assignment policy."""
    schedule = pick_schedule(schedule)
    from thor_megakernels_b200.demos.latency.scheduler import LatencyScheduleBuilder, build_b200_schedule
    from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    if schedule == "b200":
        return build_b200_schedule(model, **kwargs)
    sched = LatencyScheduleBuilder.build(model, **kwargs)
    tensorize_instructions(sched.globs, assign_to_sms(schedule, schedule=sched))
    return sched


def build_gpu_model(device, schedule: str = "b200"):
    from thor_megakernels_b200.demos.latency.scheduler import LatencyScheduleBuilder
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig
    from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    extra = ExtraModelConfig(interleave_rope=True, max_len_override=PROMPT_LEN + TOKENS_PER_REQUEST + 12)
    model = LlamaForCausalLM.random_init(LlamaConfig(**MODEL), extra, seed=0, device=device, generate_on=device)
    gen = torch.Generator(device=device).manual_seed(3)
    for cache in model.stacked_kv_cache:
        cache[:, :, :PROMPT_LEN] = torch.randn(cache[:, :, :PROMPT_LEN].shape, generator=gen, device=device).bfloat16()
    return model, make_schedule(model, schedule)


def time_cpu_oracle(model_gpu, tokens: int, threads: int, warm: int = 1):
    """Seconds per token of the CPU interpreter on a copy of the GPU model's weights."""
    from oracle import pyvm
    from thor_megakernels_b200.demos.latency.scheduler import LatencyScheduleBuilder
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig

    torch.set_num_threads(threads)
    extra = ExtraModelConfig(interleave_rope=True, max_len_override=PROMPT_LEN + TOKENS_PER_REQUEST + 12)
    if model_gpu is not None:
        # same weights as the GPU arm: clone its finalised tensors to the host
        prev = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        try:
            with torch.device("meta"):
                cpu = LlamaForCausalLM(LlamaConfig(**MODEL), extra)
        finally:
            torch.set_default_dtype(prev)
        cpu.device, cpu.dtype = torch.device("cpu"), torch.bfloat16
        sd = {k: v.detach().to("cpu") for k, v in model_gpu.state_dict().items()}
        cpu.load_state_dict(sd, strict=False, assign=True)
        if MODEL.get("tie_word_embeddings", True):
            cpu.lm_head.lm_head.weight = cpu.model.embed_tokens.embed_tokens.weight
        cpu.model.rope_cos = model_gpu.model.rope_cos.cpu()
        cpu.model.rope_sin = model_gpu.model.rope_sin.cpu()
        cpu.requires_grad_(False)
        cpu.stack_params()
        cpu.setup_caches()
        for dst, src in zip(cpu.stacked_kv_cache, model_gpu.stacked_kv_cache):
            dst.copy_(src.cpu())
    else:
        cpu = LlamaForCausalLM.random_init(LlamaConfig(**MODEL), extra, seed=0, device="cpu")
    sched = LatencyScheduleBuilder.build(cpu)
    instr = sched.get_linear_instructions()
    tok = torch.tensor([[17]])
    times = []
    for i in range(warm + tokens):
        t0 = time.perf_counter()
        tok = pyvm.pyvm_step(cpu, sched, instr, tok.view(1, 1), PROMPT_LEN + i).view(1, 1)
        if i >= warm:
            times.append(time.perf_counter() - t0)
    return times


def run_reference(args, rank, world):
    """The reference's CPU path for this workload: its PyTorch interpreter of the
    instruction stream (restated under oracle/), all host threads, one decode
    token per step."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    model_gpu = None
    if torch.cuda.is_available():
        model_gpu, _ = build_gpu_model("cuda:0")
    times = time_cpu_oracle(model_gpu, args.steps, threads, warm=args.warmup)
    total = sum(times)
    tps = len(times) / total
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * total / len(times),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": HEADLINE_WORKLOAD,
                   "step": "one decode token on the host cores (bounded sample of the 100-token request)"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{len(times)} decode tokens of the 16-layer model, PyTorch interpreter, {threads} threads"},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank, world, local):
    from thor_megakernels_b200.generators import MK_FusedGenerator

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py measures the CUDA megakernel; no CUDA device is visible")
    device = torch.device(f"cuda:{local}")
    torch.cuda.set_device(device)
    model, sched = build_gpu_model(device, schedule=args.schedule)
    gen = MK_FusedGenerator(model, sched)
    mk = gen.mk
    stream = torch.cuda.current_stream(device)
    first = torch.tensor([17], dtype=torch.int32, device=device)
    produced = torch.zeros(TOKENS_PER_REQUEST, dtype=torch.int32, device=device)

    def request_resident():
        mk.decode(first, produced, start_pos=PROMPT_LEN, count=TOKENS_PER_REQUEST, stream=stream)

    for _ in range(max(args.warmup, 3)):
        request_resident()
    torch.cuda.synchronize(device)
    mk.status()

    sampler = ClockSampler(local)
    barrier(world)
    torch.cuda.synchronize(device)
    sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(args.steps):
        request_resident()
    end.record(stream)
    torch.cuda.synchronize(device)
    barrier(world)
    clocks = sampler.stop()
    mk.status()
    elapsed_ms = max_over_ranks(start.elapsed_time(end), world)
    launches = args.steps * TOKENS_PER_REQUEST
    ms_per_step = elapsed_ms / args.steps
    tokens_per_s = world * launches / (elapsed_ms / 1000.0)

    # ---- end to end through Generator.generate with host buffers ----
    host_in = torch.tensor([[17] + [0] * TOKENS_PER_REQUEST], dtype=torch.long).pin_memory()
    host_out = torch.zeros((1, TOKENS_PER_REQUEST + 1), dtype=torch.long).pin_memory()
    dev_tokens = torch.zeros((1, TOKENS_PER_REQUEST + 1), dtype=torch.long, device=device)

    def request_e2e():
        dev_tokens[:, :1].copy_(host_in[:, :1], non_blocking=True)
        gen.generate(dev_tokens, prompt_len=PROMPT_LEN, ntok=TOKENS_PER_REQUEST, ntok_already_generated=1)
        host_out[:, 1:].copy_(dev_tokens[:, 1:], non_blocking=True)
        stream.synchronize()

    for _ in range(3):
        request_e2e()
    barrier(world)
    torch.cuda.synchronize(device)
    start.record(stream)
    for _ in range(args.steps):
        request_e2e()
    end.record(stream)
    torch.cuda.synchronize(device)
    e2e_ms = max_over_ranks(start.elapsed_time(end), world)
    e2e_tps = world * launches / (e2e_ms / 1000.0)
    assert torch.equal(host_out[0, 1:].to(torch.int32), produced.cpu()), "e2e and resident loops disagree"

    line = None
    if rank == 0:
        peak, peak_src = measured_hbm_peak()
        bytes_per_launch = algorithmic_bytes_per_request(MODEL) / TOKENS_PER_REQUEST
        launch_ms = elapsed_ms / launches
        achieved = bytes_per_launch / (launch_ms / 1000.0) / 1e9
        line = {
            "metric": "decode_tokens_per_s", "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": ("SELF-TEST (2 layers, small vocabulary) - not the benchmark workload" if args.self_test else
                             HEADLINE_WORKLOAD),
                "step": "one 100-token request = 100 megakernel launches",
                "ms_per_token": launch_ms,
                "l2": "inputs larger than L2 (2.47 GB of weights streamed per launch vs 126 MB)",
                "parallelism": "single",
                "schedule": f"reference latency instruction set, layout/policy {pick_schedule(args.schedule)}, one queue per SM",
            },
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": MEASURED_DRAM_TRAFFIC_PER_LAUNCH, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": bytes_per_launch, "launch_ms": launch_ms,
                         "frac_of_nominal_8TBs": achieved / 8000.0},
            "e2e": {"value": e2e_tps, "unit": "tokens/s", "h2d_bytes_per_step": 8,
                    "d2h_bytes_per_step": 8 * TOKENS_PER_REQUEST, "api": "MK_FusedGenerator.generate",
                    "ms_per_token": e2e_ms / launches},
            "gpu_launches": launches,
            "clocks": clocks,
        }
    # CPU baseline: rank 0, single-GPU runs only
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        times = time_cpu_oracle(model, args.cpu_tokens, threads)
        line["cpu_baseline"] = {"value": len(times) / sum(times), "unit": "tokens/s", "cores": threads, "kind": "port",
                                "sample": f"{len(times)} decode tokens of the same 16-layer model through the CPU "
                                          f"interpreter (oracle/pyvm.py), {threads} threads"}
    elif rank == 0:
        line["cpu_baseline"] = None
    if not args.no_8b and not args.self_test:
        # the 1-GPU point of the Llama-3.1-8B curve; the 1B model is dropped first
        gen.mk.close()
        del gen, mk, model, sched
        torch.cuda.empty_cache()
        line["llama8b_tp"] = llama8b_records(args, rank, world, local)
    if rank == 0:
        print(json.dumps(line), flush=True)


def run_gemv(args, rank, world, local):
    """Single-operator GEMV (bf16 and NVFP4 weight-only, batch 1 and 4) at the two
    shapes of the 1B FFN.  A call streams 9-34 MB, less than L2 holds, so every
    call uses the next of enough independently quantised weight copies to exceed
    L2 (~300 MB per case): each weight byte comes from HBM.  128 calls are
    captured in one CUDA graph so that launch latency (about the kernel's own
    duration) stays out of the figure."""
    if rank != 0:
        return
    from thor_megakernels_b200 import nvfp4

    device = torch.device(f"cuda:{local}")
    torch.cuda.set_device(device)
    peak, peak_src = measured_hbm_peak()
    gen = torch.Generator(device=device).manual_seed(2)
    calls = 128
    results = []
    for m, k in ((8192, 2048), (2048, 8192)):
        for fmt in ("nvfp4", "bf16"):
            per_weight = 0.5625 if fmt == "nvfp4" else 2.0
            copies = max(2, int(300e6 / (m * k * per_weight)) + 1)
            weights = []
            for _ in range(copies):
                w = (torch.randn(m, k, device=device, generator=gen) * 0.02).bfloat16()
                weights.append(nvfp4.quantize_weight(w) if fmt == "nvfp4" else w)
            for batch in (1, 4):
                x = torch.randn(batch, k, device=device, generator=gen).bfloat16()
                y = torch.empty(batch, m, dtype=torch.bfloat16, device=device)
                nvfp4.gemv(weights[0], x, out=y)  # first call outside capture (allocates the split-K scratch)
                torch.cuda.synchronize(device)
                stream = torch.cuda.Stream(device)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.stream(stream):
                    for i in range(3):
                        nvfp4.gemv(weights[i % copies], x, out=y)
                    stream.synchronize()
                    with torch.cuda.graph(graph, stream=stream):
                        for i in range(calls):
                            nvfp4.gemv(weights[i % copies], x, out=y)
                    for _ in range(max(args.warmup, 3)):
                        graph.replay()
                    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record(stream)
                    for _ in range(args.steps):
                        graph.replay()
                    end.record(stream)
                    stream.synchronize()
                us = 1000.0 * start.elapsed_time(end) / (args.steps * calls)
                weight_bytes = m * k * per_weight
                gbs = weight_bytes / (us * 1e-6) / 1e9
                results.append({"m": m, "k": k, "weights": fmt, "batch": batch, "us_per_call": us, "GB/s": gbs,
                                "frac_of_measured_peak": gbs / peak, "weight_copies_cycled": copies})
    best = max(results, key=lambda r: r["GB/s"])
    line = {
        "metric": "gemv_weight_GBps", "value": best["GB/s"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 activations, NVFP4 or bf16 weights", "data": "synthetic",
        "config": {"workload": "single-operator GEMV, shapes 8192x2048 and 2048x8192, batch 1 and 4",
                   "l2": "weight copies cycled so that every call reads from HBM (footprint ~300 MB per case > 126 MB L2)",
                   "timing": f"{calls} calls per CUDA graph replay, CUDA events around {args.steps} replays"},
        "roofline": {"bound": "hbm", "achieved": best["GB/s"], "peak": peak, "unit": "GB/s", "frac": best["GB/s"] / peak,
                     "traffic": None, "peak_source": peak_src},
        "cases": results, "gpu_launches": args.steps * calls * len(results), "cpu_baseline": None,
    }
    print(json.dumps(line), flush=True)


def run_long_context(args, rank, world, local):
    """Llama-3.2-1B architecture with 4096 cached positions, 256 tokens per step:
    NVFP4 weight-only against bf16 weights on the same schedule (one GPU)."""
    if rank != 0:
        return
    from thor_megakernels_b200 import nvfp4
    from thor_megakernels_b200.demos.latency.scheduler import LatencyScheduleBuilder, pick_num_attention_partitions
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig
    from thor_megakernels_b200.runtime import Megakernel
    from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    device = torch.device(f"cuda:{local}")
    torch.cuda.set_device(device)
    cfg = dict(MODEL)
    ctx, ntok = 4096, 256
    extra = ExtraModelConfig(interleave_rope=True, max_len_override=ctx + ntok + 8)
    model = LlamaForCausalLM.random_init(LlamaConfig(**cfg), extra, seed=0, device=device, generate_on=device)
    gen = torch.Generator(device=device).manual_seed(3)
    for cache in model.stacked_kv_cache:
        cache[:, :, :ctx] = torch.randn(cache[:, :, :ctx].shape, generator=gen, device=device).bfloat16()
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    partitions = min(pick_num_attention_partitions(ctx, ntok), max(1, sms // cfg["num_key_value_heads"]))
    peak, peak_src = measured_hbm_peak()
    kv = kv_bytes_per_position(cfg)
    kv_bytes = sum(kv * (pos + 1) + kv for pos in range(ctx, ctx + ntok)) / ntok
    stream = torch.cuda.current_stream(device)
    first = torch.tensor([17], dtype=torch.int32, device=device)
    produced = torch.zeros(ntok, dtype=torch.int32, device=device)
    out = {}
    for fmt in ("bf16", "nvfp4"):
        quantized = nvfp4.quantize_model(model) if fmt == "nvfp4" else None
        sched = make_schedule(model, pick_schedule(args.schedule, fmt), skip_attn_reduction=False,
                              num_attention_partitions=partitions)
        mk = Megakernel.from_globals(sched.globs, embed_w=model.model.embed_tokens.embed_tokens.weight.data, quantized=quantized)
        sched.globs.barriers.zero_()
        for _ in range(max(args.warmup, 3)):
            mk.decode(first, produced, start_pos=ctx, count=ntok, stream=stream)
        torch.cuda.synchronize(device)
        mk.status()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(args.steps):
            mk.decode(first, produced, start_pos=ctx, count=ntok, stream=stream)
        end.record(stream)
        torch.cuda.synchronize(device)
        mk.status()
        ms = start.elapsed_time(end) / (args.steps * ntok)
        weights = linear_weight_bytes(cfg) * (0.5625 / 2.0 if fmt == "nvfp4" else 1.0)
        gbs = (weights + kv_bytes) / (ms * 1e-3) / 1e9
        out[fmt] = {"ms_per_token": ms, "tokens_per_s": 1000.0 / ms, "algorithmic_bytes_per_launch": weights + kv_bytes,
                    "GB/s": gbs, "frac_of_measured_peak": gbs / peak}
        mk.close()
    line = {
        "metric": "decode_tokens_per_s", "value": out["nvfp4"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": out["nvfp4"]["ms_per_token"] * ntok,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations and KV, NVFP4 weights",
        "data": "synthetic",
        "config": {"workload": f"llama-3.2-1b-arch, every linear NVFP4 weight-only, {ctx} cached positions, {ntok} tokens per step",
                   "attention_partitions_per_kv_head": partitions, "l2": "inputs larger than L2"},
        "roofline": {"bound": "hbm", "achieved": out["nvfp4"]["GB/s"], "peak": peak, "unit": "GB/s",
                     "frac": out["nvfp4"]["GB/s"] / peak, "traffic": None, "peak_source": peak_src},
        "bf16_same_context": out["bf16"], "nvfp4": out["nvfp4"],
        "nvfp4_speedup_over_bf16": out["bf16"]["ms_per_token"] / out["nvfp4"]["ms_per_token"],
        "gpu_launches": 2 * args.steps * ntok, "cpu_baseline": None,
    }
    print(json.dumps(line), flush=True)


def measure_split_decode(workload: str, weights: str, steps: int, warmup: int, rank: int, world: int, local: int,
                         schedule: str = "b200", self_test: bool = False, e2e: bool = True) -> dict | None:
    """One sequence decoded with the model split over the ranks (world == 1: the
    whole model on one GPU).  Every rank calls this; rank 0 gets the record."""
    from thor_megakernels_b200.demos.latency.scheduler import LatencyScheduleBuilder, pick_num_attention_partitions
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig
    from thor_megakernels_b200.runtime import Megakernel
    from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions
    from thor_megakernels_b200.tp import TensorParallelDecoder

    cfg, ctx, ntok, seed = TP_WORKLOADS[workload]
    if self_test:
        cfg = dict(cfg, num_hidden_layers=2, vocab_size=4096)
    device = torch.device(f"cuda:{local}")
    torch.cuda.set_device(device)
    extra = ExtraModelConfig(interleave_rope=True, max_len_override=ctx + ntok + 8)
    # the device generator draws the same stream on every GPU, so all ranks hold the same model
    model = LlamaForCausalLM.random_init(LlamaConfig(**cfg), extra, seed=seed, device=device, generate_on=device)
    gen = torch.Generator(device=device).manual_seed(3)
    for cache in model.stacked_kv_cache:
        cache[:, :, :ctx] = torch.randn(cache[:, :, :ctx].shape, generator=gen, device=device).bfloat16()
    # split the cache of every KV head into as many slices as there are SMs to take them (at most 24 per
    # head, at least 256 positions each), so that one wave of attention instructions covers the GPU
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    kv_heads_here = cfg["num_key_value_heads"] // world
    partitions = min(pick_num_attention_partitions(ctx, ntok), max(1, sms // kv_heads_here)) if ctx >= 512 else 1
    fp4 = weights == "nvfp4"
    embed = model.model.embed_tokens.embed_tokens.weight.data
    if world > 1:
        dec = TensorParallelDecoder(model, rank, world, schedule=pick_schedule(schedule, weights),
                                    num_attention_partitions=partitions, nvfp4_weights=fp4)
        mk = dec.mk
        del model  # every rank keeps only its shard (and the embedding table)
    else:
        from thor_megakernels_b200 import nvfp4

        sched = make_schedule(model, pick_schedule(schedule, weights), skip_attn_reduction=partitions == 1,
                              num_attention_partitions=partitions)
        mk = Megakernel.from_globals(sched.globs, embed_w=embed, quantized=nvfp4.quantize_model(model) if fp4 else None)
        sched.globs.barriers.zero_()
    stream = torch.cuda.current_stream(device)
    first = torch.tensor([17], dtype=torch.int32, device=device)
    produced = torch.zeros(ntok, dtype=torch.int32, device=device)

    def request():
        mk.decode(first, produced, start_pos=ctx, count=ntok, stream=stream)

    for _ in range(max(warmup, 3)):
        request()
    torch.cuda.synchronize(device)
    mk.status()
    sampler = ClockSampler(local)
    barrier(world)
    torch.cuda.synchronize(device)
    sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(steps):
        request()
    end.record(stream)
    torch.cuda.synchronize(device)
    barrier(world)
    clocks = sampler.stop()
    mk.status()
    elapsed_ms = max_over_ranks(start.elapsed_time(end), world)
    launches = steps * ntok
    e2e_ms = None
    if e2e:
        host_first = torch.tensor([17], dtype=torch.int32).pin_memory()
        host_out = torch.zeros(ntok, dtype=torch.int32).pin_memory()

        def request_e2e():
            first.copy_(host_first, non_blocking=True)
            mk.decode(first, produced, start_pos=ctx, count=ntok, stream=stream)
            host_out.copy_(produced, non_blocking=True)
            stream.synchronize()

        for _ in range(2):
            request_e2e()
        barrier(world)
        torch.cuda.synchronize(device)
        start.record(stream)
        for _ in range(steps):
            request_e2e()
        end.record(stream)
        torch.cuda.synchronize(device)
        e2e_ms = max_over_ranks(start.elapsed_time(end), world)
    if world > 1:
        import torch.distributed as dist

        tokens = torch.zeros(world * ntok, dtype=torch.int32, device=device)
        dist.all_gather_into_tensor(tokens, produced)
        assert all(torch.equal(tokens[r * ntok:(r + 1) * ntok], produced) for r in range(world)), "ranks produced different tokens"
    mk.close()
    if rank != 0:
        return None
    peak, peak_src = measured_hbm_peak()
    kv = kv_bytes_per_position(cfg)
    weight_bytes = linear_weight_bytes(cfg) * (0.5625 / 2.0 if fp4 else 1.0)
    total_bytes = sum(weight_bytes + kv * (pos + 1) + kv for pos in range(ctx, ctx + ntok)) / ntok
    launch_ms = elapsed_ms / launches
    achieved = total_bytes / world / (launch_ms / 1000.0) / 1e9  # per GPU: every rank streams 1/world of the bytes
    line = {
        "metric": "decode_tokens_per_s", "value": launches / (elapsed_ms / 1000.0), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": elapsed_ms / steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16 activations and KV, NVFP4 weights" if fp4 else "bf16", "data": "synthetic",
        "config": {
            "workload": f"{workload} ({weights} weights): {'SELF-TEST 2-layer ' if self_test else ''}batch-1 greedy decode, "
                        f"{ctx} cached positions, {ntok} tokens per step",
            "step": f"{ntok} megakernel launches per rank",
            "ms_per_token": launch_ms,
            "parallelism": f"tp{world}" if world > 1 else "single",
            "attention_partitions_per_kv_head": partitions,
            "schedule": pick_schedule(schedule, weights),
            "l2": "inputs larger than L2",
        },
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": peak_src, "algorithmic_bytes_per_launch": total_bytes / world,
                     "launch_ms": launch_ms, "frac_of_nominal_8TBs": achieved / 8000.0,
                     "note": "per GPU: total algorithmic bytes / n_gpus over the launch time"},
        "gpu_launches": launches, "clocks": clocks, "cpu_baseline": None,
    }
    if e2e_ms is not None:
        line["e2e"] = {"value": launches / (e2e_ms / 1000.0), "unit": "tokens/s", "h2d_bytes_per_step": 4,
                       "d2h_bytes_per_step": 4 * ntok, "api": "Megakernel.decode on every rank",
                       "ms_per_token": e2e_ms / launches}
    return line


def run_tp(args, rank, world, local):
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py measures the CUDA megakernel; no CUDA device is visible")
    line = measure_split_decode(args.workload, args.weights, args.steps, args.warmup, rank, world, local,
                                schedule=args.schedule, self_test=args.self_test)
    if rank == 0:
        print(json.dumps(line), flush=True)


PARITY_MODEL = dict(hidden_size=2048, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
                    intermediate_size=8192, vocab_size=4096)


def tp_parity_check(rank: int, world: int, local: int) -> dict | None:
    """Four tokens of a 2-layer model, decoded with the model split over the ranks
    and, on rank 0, with the whole model on one GPU fed the same tokens.  The
    split sums in a different order, so hidden state and logits agree to the
    rounding noise of two layers (NRMSE about 1 %), not bit for bit; the ranks
    among themselves must be bit-identical."""
    import torch.distributed as dist

    from thor_megakernels_b200.demos.latency.scheduler import LatencyScheduleBuilder
    from thor_megakernels_b200.dispatch import make_mk_interpreter
    from thor_megakernels_b200.generators import MK_Generator
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig
    from thor_megakernels_b200.scheduler import assign_to_sms, tensorize_instructions
    from thor_megakernels_b200.tp import TensorParallelDecoder

    device = torch.device(f"cuda:{local}")
    ctx, ntok, first = 19, 4, 77
    model = LlamaForCausalLM.random_init(LlamaConfig(**PARITY_MODEL), ExtraModelConfig(interleave_rope=True, max_len_override=64),
                                         seed=3, device=device, generate_on=device)
    gen = torch.Generator(device=device).manual_seed(21)
    for cache in model.stacked_kv_cache:
        cache[:, :, :ctx] = torch.randn(cache[:, :, :ctx].shape, generator=gen, device=device).bfloat16()
    tp = TensorParallelDecoder(model, rank, world)
    tokens = tp.decode(first, ntok, ctx)
    torch.cuda.synchronize(device)
    tp.mk.status()
    hidden = tp.schedule.globs.hidden_states.clone()
    vocab_share = PARITY_MODEL["vocab_size"] // world
    logits = torch.empty(world * vocab_share, dtype=torch.bfloat16, device=device)
    dist.all_gather_into_tensor(logits, tp.logits().contiguous())
    all_hidden = torch.empty(world * hidden.numel(), dtype=torch.bfloat16, device=device)
    dist.all_gather_into_tensor(all_hidden, hidden)
    all_tokens = torch.empty(world * ntok, dtype=torch.int32, device=device)
    dist.all_gather_into_tensor(all_tokens, tokens)
    identical = all(torch.equal(all_hidden[r * hidden.numel():(r + 1) * hidden.numel()], hidden) and
                    torch.equal(all_tokens[r * ntok:(r + 1) * ntok], tokens) for r in range(world))
    out = None
    if rank == 0:
        sched = LatencyScheduleBuilder.build(model)
        tensorize_instructions(sched.globs, assign_to_sms("rr", schedule=sched))
        whole = MK_Generator(model, make_mk_interpreter("latency"), sched)
        fed = [first] + tokens.cpu().tolist()[:-1]
        whole_tokens = [int(whole.run(torch.tensor([[tok]], device=device), pos_id=ctx + i)) for i, tok in enumerate(fed)]
        torch.cuda.synchronize(device)
        g = sched.globs

        def nrmse(a, b):
            a, b = a.float(), b.float()
            return float((a - b).norm() / b.norm().clamp_min(1e-12))

        out = {"model": "2 layers of the 1B shapes, 4 tokens, split over the ranks vs whole on rank 0 (teacher-forced)",
               "nrmse_hidden": nrmse(hidden, g.hidden_states), "nrmse_logits": nrmse(logits, g.logits),
               "tokens_equal": sum(int(a == b) for a, b in zip(tokens.cpu().tolist(), whole_tokens)), "tokens": ntok,
               "ranks_bit_identical": bool(identical),
               "ok": bool(identical) and nrmse(hidden, g.hidden_states) <= 0.02 and nrmse(logits, g.logits) <= 0.02}
    tp.close()
    dist.barrier()
    return out


def llama8b_records(args, rank, world, local) -> dict | None:
    """Config-4 figures at this GPU count: bf16 and NVFP4 weight-only."""
    out = {}
    steps = max(2, min(args.steps, 6))
    for weights in ("bf16", "nvfp4"):
        line = measure_split_decode("llama8b-tp", weights, steps, 3, rank, world, local, schedule=args.schedule,
                                    self_test=args.self_test, e2e=False)
        torch.cuda.empty_cache()
        if rank == 0:
            out[weights] = {"tokens_per_s": line["value"], "ms_per_token": line["config"]["ms_per_token"],
                            "per_gpu_roofline_frac": line["roofline"]["frac"], "per_gpu_GBps": line["roofline"]["achieved"],
                            "attention_partitions_per_kv_head": line["config"]["attention_partitions_per_kv_head"],
                            "clocks": line["clocks"], "steps": steps, "tokens_per_step": TP_WORKLOADS["llama8b-tp"][2]}
    if rank != 0:
        return None
    out["workload"] = ("llama-3.1-8b-arch batch-1 greedy decode, 8192 cached positions, 64 tokens per step, "
                       f"{'split over ' + str(world) + ' GPUs (tensor parallel)' if world > 1 else 'one GPU'}")
    return out


def run_headline_split(args, rank, world, local):
    """N > 1: the headline request with the 1B model split over the N GPUs."""
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py measures the CUDA megakernel; no CUDA device is visible")
    parity = tp_parity_check(rank, world, local)
    torch.cuda.empty_cache()
    line = measure_split_decode("llama1b-tp", "bf16", args.steps, args.warmup, rank, world, local,
                                schedule=args.schedule, self_test=args.self_test)
    torch.cuda.empty_cache()
    big = None if args.no_8b else llama8b_records(args, rank, world, local)
    if rank == 0:
        if not args.self_test:
            line["config"]["workload"] = HEADLINE_WORKLOAD   # the same request at every N; config.parallelism says how it is split
        line["tp_parity"] = parity
        line["llama8b_tp"] = big
        print(json.dumps(line), flush=True)


def build_step_model(args, device):
    """Model + schedule of the timeline / profile-step workloads: the headline 1B
    model (``--layers`` shrinks it), or with ``--arch 8b`` a few layers of the
    Llama-3.1-8B shapes with ``--pos`` cached positions split into
    ``--partitions`` attention slices per KV head."""
    if args.arch == "8b":
        from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
        from thor_megakernels_b200.model_types import ExtraModelConfig

        cfg = dict(MODEL_8B, num_hidden_layers=args.layers or 4)
        extra = ExtraModelConfig(interleave_rope=True, max_len_override=args.pos + 16)
        model = LlamaForCausalLM.random_init(LlamaConfig(**cfg), extra, seed=4, device=device, generate_on=device)
        gen = torch.Generator(device=device).manual_seed(3)
        for cache in model.stacked_kv_cache:
            cache[:, :, :args.pos] = torch.randn(cache[:, :, :args.pos].shape, generator=gen, device=device).bfloat16()
        sched = make_schedule(model, pick_schedule(args.schedule, args.weights), skip_attn_reduction=args.partitions == 1,
                              num_attention_partitions=args.partitions)
        sched.globs.barriers.zero_()
        return model, sched, cfg
    if args.layers is not None:
        MODEL.update(num_hidden_layers=args.layers)
    model, sched = build_gpu_model(device, schedule=pick_schedule(args.schedule, args.weights))
    return model, sched, dict(MODEL)


def run_batched(args, rank, world, local):
    """Batched decode (config 3): the 1B architecture, 16 / 64 / 128 sequences
    with independent cache lengths drawn uniformly from [512, 4096] (seed 3),
    128 greedy steps per measurement, linears on the tcgen05 tensor cores.  A
    step is captured once in a CUDA graph (about 165 launches) and replayed; the
    positions advance on the device between replays."""
    if rank != 0:
        return
    from thor_megakernels_b200.batched import BatchedDecoder
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig

    device = torch.device(f"cuda:{local}")
    torch.cuda.set_device(device)
    cfg = dict(MODEL)
    steps_per_run, max_ctx = 128, 4096
    peak, peak_src = measured_hbm_peak()
    results = []
    for weights, batch in [(w, b) for w in ("bf16", "nvfp4") for b in (16, 64, 128)]:
        extra = ExtraModelConfig(interleave_rope=True, max_len_override=max_ctx + steps_per_run + 8, max_batch_size=batch)
        model = LlamaForCausalLM.random_init(LlamaConfig(**cfg), extra, seed=0, device=device, generate_on=device)
        gen = torch.Generator().manual_seed(3)
        lengths = torch.randint(512, max_ctx + 1, (batch,), generator=gen)
        dgen = torch.Generator(device=device).manual_seed(3)
        for cache in model.stacked_kv_cache:
            for b in range(batch):
                n = int(lengths[b])
                cache[:, b, :n] = torch.randn(cache[:, b, :n].shape, generator=dgen, device=device).bfloat16()
        quantized = None
        if weights == "nvfp4":
            from thor_megakernels_b200.nvfp4 import quantize_model

            quantized = quantize_model(model)
        dec = BatchedDecoder(model, batch, quantized=quantized)
        tokens = torch.randint(0, cfg["vocab_size"], (batch,), generator=gen).int().to(device)
        start_pos = lengths.int().to(device)
        pos = start_pos.clone()
        out = torch.zeros(batch, dtype=torch.int32, device=device)
        stream = torch.cuda.Stream(device)
        with torch.cuda.stream(stream):
            dec.step(tokens, pos, out)   # outside capture once
            stream.synchronize()
            dec.status()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                dec.step(tokens, pos, out)
                tokens.copy_(out)
                pos.add_(1)

            def run():
                pos.copy_(start_pos)
                for _ in range(steps_per_run):
                    graph.replay()

            for _ in range(max(args.warmup, 3) if args.steps > 2 else 1):
                run()
            stream.synchronize()
            dec.status()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(1, min(args.steps, 5))
            start.record(stream)
            for _ in range(reps):
                run()
            end.record(stream)
            stream.synchronize()
        dec.status()
        ms_per_step = start.elapsed_time(end) / (reps * steps_per_run)
        kv = kv_bytes_per_position(cfg)
        kv_bytes = float(sum(kv * (int(n) + steps_per_run / 2 + 1) for n in lengths))   # mean over the run's positions
        weight_bytes = linear_weight_bytes(cfg) * (0.5625 / 2.0 if weights == "nvfp4" else 1.0)
        gbs = (weight_bytes + kv_bytes) / (ms_per_step * 1e-3) / 1e9
        flops = 2.0 * batch * (linear_weight_bytes(cfg) / 2)
        results.append({"weights": weights, "batch": batch, "ms_per_step": ms_per_step, "tokens_per_s": batch / (ms_per_step * 1e-3),
                        "algorithmic_bytes_per_step": weight_bytes + kv_bytes, "kv_share": kv_bytes / (weight_bytes + kv_bytes),
                        "GB/s": gbs, "frac_of_measured_peak": gbs / peak, "linear_TFLOPs": flops / (ms_per_step * 1e-3) / 1e12,
                        "mean_cache_length": float(lengths.float().mean())})
        dec.close()
        del dec, model, quantized
        torch.cuda.empty_cache()
    best = max((r for r in results if r["weights"] == "bf16"), key=lambda r: r["tokens_per_s"])
    line = {"metric": "decode_tokens_per_s", "value": best["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": best["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "llama-3.2-1b-arch batched greedy decode, 16/64/128 sequences, cache lengths uniform in "
                                   "[512, 4096] (seed 3), 128 steps per run, bf16 weights and (cases) NVFP4 weights + activations; "
                                   "value = best bf16 batch size",
                       "step": "one decode step for the whole batch = one CUDA graph replay (tcgen05 linears + batched attention)",
                       "l2": "inputs larger than L2 (weights 2.47 GB + KV 0.6-9.7 GB per step)"},
            "roofline": {"bound": "hbm", "achieved": best["GB/s"], "peak": peak, "unit": "GB/s", "frac": best["GB/s"] / peak,
                         "traffic": None, "peak_source": peak_src},
            "cases": results, "gpu_launches": None, "cpu_baseline": None}
    print(json.dumps(line), flush=True)


def run_batched_step(args, rank, world, local):
    """A few plain (not graph-captured) batched decode steps at one batch size, for a
    profiler's launch list: --batch sequences, cache lengths as in llama1b-batched,
    optionally fewer layers (--layers) and NVFP4 weights and activations (--weights nvfp4)."""
    if rank != 0:
        return
    from thor_megakernels_b200.batched import BatchedDecoder
    from thor_megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
    from thor_megakernels_b200.model_types import ExtraModelConfig

    device = torch.device(f"cuda:{local}")
    torch.cuda.set_device(device)
    cfg = dict(MODEL)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    batch, max_ctx = args.batch, 4096
    extra = ExtraModelConfig(interleave_rope=True, max_len_override=max_ctx + args.steps + args.warmup + 8, max_batch_size=batch)
    model = LlamaForCausalLM.random_init(LlamaConfig(**cfg), extra, seed=0, device=device, generate_on=device)
    gen = torch.Generator().manual_seed(3)
    lengths = torch.randint(512, max_ctx + 1, (batch,), generator=gen)
    dgen = torch.Generator(device=device).manual_seed(3)
    for cache in model.stacked_kv_cache:
        for b in range(batch):
            n = int(lengths[b])
            cache[:, b, :n] = torch.randn(cache[:, b, :n].shape, generator=dgen, device=device).bfloat16()
    quantized = None
    if args.weights == "nvfp4":
        from thor_megakernels_b200.nvfp4 import quantize_model

        quantized = quantize_model(model)
    dec = BatchedDecoder(model, batch, quantized=quantized)
    tokens = torch.randint(0, cfg["vocab_size"], (batch,), generator=gen).int().to(device)
    pos = lengths.int().to(device)
    out = torch.zeros(batch, dtype=torch.int32, device=device)
    for _ in range(args.warmup):
        dec.step(tokens, pos, out)
        pos.add_(1)
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        dec.step(tokens, pos, out)
        pos.add_(1)
    end.record()
    torch.cuda.synchronize(device)
    dec.status()
    print(json.dumps({"workload": f"batched decode step, {batch} sequences, {cfg['num_hidden_layers']} layers, {args.weights}, "
                                  "plain launches (no CUDA graph)",
                      "ms_per_step": start.elapsed_time(end) / args.steps, "steps": args.steps, "warmup": args.warmup}), flush=True)


def run_timeline(args, rank, world, local):
    """One decode step with per-instruction clock stamps; prints, per opcode of a
    middle layer, when its instructions had their input, how long they streamed
    and when their output was stored, plus the hand-off gaps between phases."""
    if rank != 0:
        return
    import numpy as np

    from thor_megakernels_b200.runtime import (MK_STEP_EMBED, MK_STEP_RESET_BARRIERS, MK_STEP_TIMINGS, MK_STEP_WRITE_TOKEN,
                                               Megakernel)

    device = torch.device(f"cuda:{local}")
    torch.cuda.set_device(device)
    model, sched, cfg = build_step_model(args, device)
    g = sched.globs
    quantized = None
    if args.weights == "nvfp4":
        from thor_megakernels_b200.nvfp4 import quantize_model

        quantized = quantize_model(model)
    mk = Megakernel.from_globals(g, embed_w=model.model.embed_tokens.embed_tokens.weight.data, quantized=quantized)
    tok = torch.tensor([17], dtype=torch.int32, device=device)
    out = torch.zeros(1, dtype=torch.int32, device=device)
    flags = MK_STEP_EMBED | MK_STEP_RESET_BARRIERS | MK_STEP_WRITE_TOKEN
    for _ in range(5):
        mk.step(args.pos, flags=flags, token_in=tok, token_out=out)
    torch.cuda.synchronize(device)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    mk.step(args.pos, flags=flags, token_in=tok, token_out=out)
    e.record()
    torch.cuda.synchronize(device)
    plain_ms = s.elapsed_time(e)
    g.timings.zero_()
    s.record()
    mk.step(args.pos, flags=flags | MK_STEP_TIMINGS, token_in=tok, token_out=out)
    e.record()
    torch.cuda.synchronize(device)
    mk.status()
    stamped_ms = s.elapsed_time(e)
    T, I = g.timings.cpu().numpy().astype(np.float64), g.instructions.cpu().numpy()
    mhz = torch.cuda.clock_rate() if hasattr(torch.cuda, "clock_rate") else 1965
    T = T / float(mhz)  # microseconds since the CTA started
    ops = I[:, :, 0]
    names = {1: "qkv", 2: "attention", 3: "attn_merge", 4: "o_proj", 5: "gate_up", 6: "down", 7: "lm_head"}
    layers = cfg["num_hidden_layers"]
    mid = list(range(max(1, layers // 2 - 2), min(layers - 1, layers // 2 + 2))) or [layers - 1]
    rows, ends = [], {}
    for op in (1, 2, 3, 4, 5, 6):
        per_layer = []
        for layer in mid:
            m = (ops == op) & (I[:, :, 1] == layer)
            if not m.any():
                continue
            ready = np.where(op == 2, T[:, :, 45], T[:, :, 49])[m]   # input present (attention: q arrived)
            last_use, last_store = T[:, :, 52][m], np.where(op in (2, 3), T[:, :, 54], T[:, :, 53])[m]
            per_sm = m.sum(axis=1)
            per_layer.append((ready.min(), ready.max(), last_use.min(), last_use.max(), last_store.max(),
                              float(np.mean(last_use - ready)), int(m.sum()), int(per_sm.max()), int((per_sm > 0).sum())))
            ends[(op, layer)] = (ready.min(), last_store.max())
        if per_layer:
            a = np.array(per_layer, dtype=np.float64)
            t0 = np.array([ends[(1, layer)][0] for layer in mid])  # relative to the layer's first QKV input
            rows.append({"op": names[op], "instructions_per_layer": int(a[0, 6]), "sms_used": int(a[0, 8]),
                         "max_instructions_per_sm": int(a[0, 7]),
                         "input_ready_us": [round(float(np.mean(a[:, 0] - t0)), 2), round(float(np.mean(a[:, 1] - t0)), 2)],
                         "last_use_us": [round(float(np.mean(a[:, 2] - t0)), 2), round(float(np.mean(a[:, 3] - t0)), 2)],
                         "output_stored_us": round(float(np.mean(a[:, 4] - t0)), 2),
                         "mean_streaming_us": round(float(np.mean(a[:, 5])), 2)})
    layer_us = float(np.mean([ends[(1, layer + 1)][0] - ends[(1, layer)][0] for layer in mid if (1, layer + 1) in ends]))
    m7 = ops == 7
    head = {"input_ready_us": [float(T[:, :, 49][m7].min()), float(T[:, :, 49][m7].max())],
            "last_use_us": [float(T[:, :, 52][m7].min()), float(T[:, :, 52][m7].max())]}
    weights_mb = (linear_weight_bytes(cfg) - 2 * cfg["vocab_size"] * cfg["hidden_size"]) / layers / 1e6
    if args.weights == "nvfp4":
        weights_mb *= 0.5625 / 2
    print(json.dumps({"workload": f"one step at position {args.pos}, {args.arch} shapes ({layers} layers), {args.weights} weights, "
                                  f"schedule {pick_schedule(args.schedule, args.weights)}",
                      "ms_plain": plain_ms, "ms_with_stamps": stamped_ms, "layers_averaged": mid,
                      "layer_period_us": round(layer_us, 2), "layer_weight_MB": round(weights_mb, 1),
                      "times": "microseconds after the layer's first QKV instruction had its input; [earliest SM, latest SM]",
                      "per_op": rows, "lm_head": head}), flush=True)
    if args.dump:
        np.savez_compressed(args.dump, timings=g.timings.cpu().numpy(), instructions=I)


def run_profile_step(args, rank, world, local):
    """A few bare decode steps and nothing else, so that a profiler sees only
    megakernel launches.  Prints the mean step time measured with CUDA events."""
    if rank != 0:
        return
    from thor_megakernels_b200.runtime import MK_STEP_EMBED, MK_STEP_RESET_BARRIERS, MK_STEP_WRITE_TOKEN, Megakernel

    device = torch.device(f"cuda:{local}")
    torch.cuda.set_device(device)
    model, sched, _ = build_step_model(args, device)
    quantized = None
    if args.weights == "nvfp4":
        from thor_megakernels_b200.nvfp4 import quantize_model

        quantized = quantize_model(model)
    mk = Megakernel.from_globals(sched.globs, embed_w=model.model.embed_tokens.embed_tokens.weight.data, quantized=quantized)
    tok = torch.tensor([17], dtype=torch.int32, device=device)
    out = torch.zeros(1, dtype=torch.int32, device=device)
    flags = MK_STEP_EMBED | MK_STEP_RESET_BARRIERS | MK_STEP_WRITE_TOKEN
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    mk.step(args.pos, flags=flags, token_in=tok, token_out=out)
    torch.cuda.synchronize(device)
    start.record()
    for _ in range(args.steps):
        mk.step(args.pos, flags=flags, token_in=tok, token_out=out)
    end.record()
    torch.cuda.synchronize(device)
    mk.status()
    print(f"{args.steps} steps at position {args.pos}: {start.elapsed_time(end) / args.steps:.4f} ms/step, token {int(out)}")


# dram__bytes_read.sum + dram__bytes_write.sum of one megakernel launch from an ncu capture
# of this workload at position 60 (summarised under profiles/).
MEASURED_DRAM_TRAFFIC_PER_LAUNCH = 2_476_319_000 + 9_706_496


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-tokens", type=int, default=4, help="decode tokens timed for cpu_baseline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-8b", action="store_true", help="leave out the nested Llama-3.1-8B record")
    ap.add_argument("--workload", default="llama1b",
                    choices=["llama1b", *TP_WORKLOADS, "gemv", "llama1b-nvfp4-4k", "llama1b-batched", "batched-step", "timeline", "profile-step"],
                    help="llama1b: the headline workload (split over the GPUs when N > 1); *-tp: only the split decode")
    ap.add_argument("--weights", default="bf16", choices=["bf16", "nvfp4"], help="weight format (tp, timeline, profile-step)")
    ap.add_argument("--schedule", default="auto", choices=["auto", "b200", "rr", "zz", "wave", "dag"],
                    help="b200: one SM owns all column slices of its down-projection rows; others: the reference's "
                         "layout under that assignment policy; auto: b200 for bf16 weights, rr for NVFP4")
    ap.add_argument("--pos", type=int, default=60, help="timeline / profile-step: position of the step")
    ap.add_argument("--layers", type=int, default=None, help="profile-step: shrink the model to this many layers")
    ap.add_argument("--arch", default="1b", choices=["1b", "8b"], help="profile-step: layer shapes")
    ap.add_argument("--partitions", type=int, default=18, help="profile-step --arch 8b: attention slices per KV head")
    ap.add_argument("--batch", type=int, default=128, help="batched-step: sequences per step")
    ap.add_argument("--dump", default=None, help="timeline: also save the raw stamps to this .npz file")
    ap.add_argument("--self-test", action="store_true",
                    help="2-layer, 4096-token-vocabulary model to exercise this script quickly; not a benchmark")
    args = ap.parse_args()
    if args.self_test:
        MODEL.update(num_hidden_layers=2, vocab_size=4096)
    rank, world, local = dist_setup(args.gpus)
    try:
        if args.impl == "reference":
            run_reference(args, rank, world)
        elif args.workload == "gemv":
            run_gemv(args, rank, world, local)
        elif args.workload == "llama1b-nvfp4-4k":
            run_long_context(args, rank, world, local)
        elif args.workload == "llama1b-batched":
            run_batched(args, rank, world, local)
        elif args.workload == "batched-step":
            run_batched_step(args, rank, world, local)
        elif args.workload == "timeline":
            run_timeline(args, rank, world, local)
        elif args.workload == "profile-step":
            run_profile_step(args, rank, world, local)
        elif args.workload != "llama1b":
            run_tp(args, rank, world, local)
        elif world > 1:
            run_headline_split(args, rank, world, local)
        else:
            run_ours(args, rank, world, local)
    finally:
        if world > 1:
            import torch.distributed as dist

            if dist.is_initialized():
                dist.destroy_process_group()


if __name__ == "__main__":
    main()
