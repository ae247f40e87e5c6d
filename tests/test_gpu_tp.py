"""Tensor-parallel decode on the GPU.

* One GPU: a rank's shard is itself a valid (narrower) model, so the kernel's
  variable tile widths (output-projection input of 256..2048 columns,
  down-projection slices of 1024 or 1792 columns) are checked against the oracle
  on the same shard, buffer by buffer.
* Two or more GPUs (skipped otherwise): the model split over the ranks with the
  in-kernel all-reduce against the whole model on one GPU.
"""
import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from helpers import assert_close, build_model, build_schedule, nrmse

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

B1 = dict(hidden_size=2048, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
          intermediate_size=8192, vocab_size=4096)
B8 = dict(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
          intermediate_size=14336, vocab_size=4096, tie_word_embeddings=False)


@pytest.mark.parametrize("cfg,world", [(B1, 2), (B1, 4), (B1, 8), (B8, 2), (B8, 8)])
def test_shard_shapes_against_the_oracle(cfg, world):
    from oracle import pyvm
    from thor_megakernels_b200.dispatch import make_mk_interpreter
    from thor_megakernels_b200.tp import shard_model

    cpu = build_model(cfg, 64, device="cpu", seed=3)
    gpu = build_model(cfg, 64, device="cuda", seed=3)
    gen = torch.Generator().manual_seed(21)
    ctx = 19
    for idx in range(2):
        kv = torch.randn(cpu.stacked_kv_cache[idx][:, :, :ctx].shape, generator=gen).bfloat16()
        cpu.stacked_kv_cache[idx][:, :, :ctx] = kv
        gpu.stacked_kv_cache[idx][:, :, :ctx] = kv.cuda()
    rank = world - 1
    cpu_shard, gpu_shard = shard_model(cpu, rank, world), shard_model(gpu, rank, world)
    # one layer, so that every buffer holds values an exact restatement also reaches within the band
    cs, gs = build_schedule(cpu_shard, layer_limit=1), build_schedule(gpu_shard, layer_limit=1)
    h0 = cpu.model.embed_tokens.embed_tokens.weight[77]
    cs.globs.hidden_states[:] = h0
    gs.globs.hidden_states[:] = h0.cuda()
    for g in (cs.globs, gs.globs):
        g.barriers.zero_()
        g.pos_id = ctx
    pyvm.interpret_with_pyvm(cs.globs, cs.get_linear_instructions())
    make_mk_interpreter("latency").interpret(gs.globs)
    torch.cuda.synchronize()
    for name in ("post_ln_rope_q", "attn_out", "silu_out", "hidden_states"):
        assert_close(name, getattr(gs.globs, name), getattr(cs.globs, name))
    assert torch.equal(gs.globs.barriers.cpu()[:, :6], cs.globs.barriers[:, :6])
    assert_close("k row", gpu_shard.stacked_kv_cache[0][0, 0, ctx], cpu_shard.stacked_kv_cache[0][0, 0, ctx])


def _run_ranks(tmp_path, world, case):
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
         "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / "tp_worker.py"), str(tmp_path), case],
        capture_output=True, text=True, env=env, timeout=900)
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-4000:])
    return [json.loads((tmp_path / f"rank{r}.json").read_text()) for r in range(world)]


@pytest.mark.parametrize("case", ["b1", "b8"])
def test_model_split_over_the_gpus_matches_the_whole_model(tmp_path, case):
    world = min(torch.cuda.device_count(), 8)
    world = 1 << (world.bit_length() - 1)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ranks = _run_ranks(tmp_path, world, case)
    r0 = ranks[0]
    assert all(r["status"] == 0 for r in ranks)
    # fixed rank-order sums: every rank holds bit-identical replicated state
    for r in ranks[1:]:
        assert r["tokens"] == r0["tokens"]
        assert r["hidden"] == r0["hidden"]
    # against the whole model on one GPU: same tolerance as against the oracle
    hidden, whole = torch.tensor(r0["hidden"]), torch.tensor(r0["whole_hidden"])
    logits = torch.cat([torch.tensor(r["logits"]) for r in ranks])
    whole_logits = torch.tensor(r0["whole_logits"])
    assert nrmse(hidden, whole) <= 0.012 * 2 ** 0.5, nrmse(hidden, whole)
    assert nrmse(logits, whole_logits) <= 0.012 * 2 ** 0.5, nrmse(logits, whole_logits)
    # the greedy token of the last step is the argmax of the gathered logits (lowest index on ties)
    assert r0["tokens"][-1] == int(torch.argmax(logits))
    # the whole model, fed the same tokens, picks the same next token except at near-ties of its top two logits
    assert sum(g != w for g, w in zip(r0["tokens"], r0["whole_tokens"])) <= 2, (r0["tokens"], r0["whole_tokens"])
    if r0["tokens"][-1] != r0["whole_tokens"][-1]:
        assert float(whole_logits[r0["whole_tokens"][-1]] - whole_logits[r0["tokens"][-1]]) < 0.25
    # appended cache rows of all layers: the ranks' KV heads side by side are the whole model's rows
    layers, ntok = 2, len(r0["tokens"])
    k = torch.cat([torch.tensor(r["k_rows"]).view(layers, ntok, -1) for r in ranks], dim=2)
    whole_k = torch.tensor(r0["whole_k_rows"]).view(layers, ntok, -1)
    assert_close("layer-0 k rows", k[0], whole_k[0])
    assert nrmse(k[1], whole_k[1]) <= 0.012 * 2 ** 0.5
