"""The multi-process plumbing of bench.py on CPU: two gloo ranks rendezvous on
127.0.0.1, take a barrier and agree on the slowest rank's time; the reference
arm only works on rank 0."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]

WORKER = r"""
import os, sys, json
sys.path.insert(0, {root!r})
import bench
rank, world, local = bench.dist_setup(2)
bench.barrier(world)
slowest = bench.max_over_ranks(10.0 + rank, world)
# one file per rank: two ranks printing to one pipe can interleave their lines
with open(os.path.join({out!r}, f"rank{{rank}}.json"), "w") as fh:
    json.dump(dict(rank=rank, world=world, slowest=slowest), fh)
import torch.distributed as dist
dist.destroy_process_group()
"""


def test_two_gloo_ranks_agree_on_the_slowest_time(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=str(ROOT), out=str(tmp_path)))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    import socket

    with socket.socket() as sock:  # a port nobody is listening on right now
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
         "127.0.0.1", "--master-port", str(port), str(script)],
        capture_output=True, text=True, env=env, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [json.loads((tmp_path / f"rank{r}.json").read_text()) for r in range(2)]
    assert sorted(l["rank"] for l in lines) == [0, 1]
    assert all(l["world"] == 2 and l["slowest"] == 11.0 for l in lines)


def test_algorithmic_byte_model():
    sys.path.insert(0, str(ROOT))
    import bench

    assert bench.linear_weight_bytes(bench.MODEL) == 2_471_493_632  # the reference's own figure for the 1B model
    assert bench.kv_bytes_per_position(bench.MODEL) == 32_768
    per_request = bench.algorithmic_bytes_per_request(bench.MODEL)
    assert per_request == sum(2_471_493_632 + 32_768 * (pos + 1) + 32_768 for pos in range(16, 116))
