"""Host side of tensor parallelism on CPU: the shard layout (reference
megakernels/llama.py:192-207, 308-310, 665-691), schedules for shard shapes, and
a two-rank gloo run in which the ranks' partial projections add up to the whole
model's."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from helpers import build_model, build_schedule

ROOT = Path(__file__).resolve().parents[1]
CFG = dict(hidden_size=2048, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
           intermediate_size=8192, vocab_size=4096)


def test_down_slice_width_rule():
    from thor_megakernels_b200.demos.latency.scheduler import down_slice_width

    assert [down_slice_width(n) for n in (8192, 14336, 7168, 3584, 1792, 4096, 1024)] == [2048, 2048, 1792, 1792, 1792, 2048, 1024]
    with pytest.raises(ValueError):
        down_slice_width(1000)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_shards_cover_every_row_once(world):
    from thor_megakernels_b200.llama import LlamaConfig
    from thor_megakernels_b200.tp import shard_slices

    cfg = LlamaConfig(**CFG)
    qkv_rows = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    seen = torch.zeros(qkv_rows, dtype=torch.int32)
    ffn = torch.zeros(cfg.intermediate_size, dtype=torch.int32)
    vocab = torch.zeros(cfg.vocab_size, dtype=torch.int32)
    for rank in range(world):
        sl = shard_slices(cfg, rank, world)
        for key in ("q_rows", "k_rows", "v_rows"):
            seen[sl[key][0]:sl[key][1]] += 1
        ffn[sl["ffn"][0]:sl["ffn"][1]] += 1
        vocab[sl["vocab"][0]:sl["vocab"][1]] += 1
        # a rank's query heads use its own KV heads (4 query heads per KV head)
        assert sl["q_rows"][0] // (4 * cfg.head_dim) == sl["kv_heads"][0]
    assert bool((seen == 1).all()) and bool((ffn == 1).all()) and bool((vocab == 1).all())


@pytest.mark.parametrize("world", [2, 4, 8])
def test_shard_partials_add_up_and_schedules_build(world):
    from thor_megakernels_b200.tp import shard_model

    model = build_model(CFG, 32, device="cpu")
    sp = model.stacked_params
    gen = torch.Generator().manual_seed(5)
    attn = torch.randn(2048, generator=gen)
    act = torch.randn(8192, generator=gen)
    o_sum, down_sum = torch.zeros(2048), torch.zeros(2048)
    for rank in range(world):
        loc = shard_model(model, rank, world)
        lsp = loc.stacked_params
        a, b = rank * 2048 // world, (rank + 1) * 2048 // world
        o_sum += lsp.o_proj[0].float() @ attn[a:b]
        f0, f1 = rank * 8192 // world, (rank + 1) * 8192 // world
        down_sum += lsp.down_proj[1].float() @ act[f0:f1]
        assert torch.equal(lsp.up_proj[1], sp.up_proj[1, f0:f1])
        sched = build_schedule(loc)
        g = sched.globs
        assert g.num_attention_heads == 32 // world and g.intermediate_size == 8192 // world
        assert g.instructions.shape[0] == 148 and g.logits.shape[0] == 4096 // world
        assert g.matvec_reduction_size * (g.intermediate_size // g.matvec_reduction_size) == g.intermediate_size
    torch.testing.assert_close(o_sum, sp.o_proj[0].float() @ attn, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(down_sum, sp.down_proj[1].float() @ act, rtol=1e-4, atol=1e-4)


WORKER = r"""
import os, sys
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
import torch, torch.distributed as dist
from helpers import build_model
from thor_megakernels_b200.tp import shard_model
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
cfg = dict(hidden_size=2048, num_hidden_layers=1, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
           intermediate_size=8192, vocab_size=4096)
model = build_model(cfg, 32, device="cpu")
loc = shard_model(model, rank, world)
x = torch.randn(2048, generator=torch.Generator().manual_seed(9))
part = loc.stacked_params.o_proj[0].float() @ x[rank * 2048 // world:(rank + 1) * 2048 // world]
dist.all_reduce(part)
full = model.stacked_params.o_proj[0].float() @ x
handles = [None] * world
dist.all_gather_object(handles, bytes([rank]) * 64)
ok = torch.allclose(part, full, rtol=1e-4, atol=1e-4) and handles == [bytes([r]) * 64 for r in range(world)]
print("TP_OK" if ok else "TP_BAD", rank, flush=True)
dist.destroy_process_group()
"""


def test_two_gloo_ranks_all_reduce_their_partials(tmp_path):
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER.format(root=str(ROOT)))
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
         "127.0.0.1", "--master-port", str(port), str(script)],
        capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.count("TP_OK") == 2, out.stdout
