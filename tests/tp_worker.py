"""One rank of the tensor-parallel GPU test (launched by tests/test_gpu_tp.py
through torch.distributed.run, one process per GPU).  Builds the same seeded
model on every rank, decodes with the model split over the ranks, and has rank 0
also decode with the whole model on its GPU; writes what it saw to a file."""
import json
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def main():
    import torch
    import torch.distributed as dist

    from helpers import build_model, build_schedule
    from thor_megakernels_b200.dispatch import make_mk_interpreter
    from thor_megakernels_b200.generators import MK_Generator
    from thor_megakernels_b200.tp import TensorParallelDecoder

    out_dir, case = Path(sys.argv[1]), sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = f"cuda:{int(os.environ['LOCAL_RANK'])}"
    dist.init_process_group("nccl")
    cfgs = {
        "b1": dict(hidden_size=2048, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
                   intermediate_size=8192, vocab_size=4096),
        "b8": dict(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                   intermediate_size=14336, vocab_size=4096, tie_word_embeddings=False),
    }
    model = build_model(cfgs[case], 64, device=dev, seed=3)
    ctx, ntok, first = 19, 6, 77
    gen = torch.Generator().manual_seed(21)
    for idx in range(2):
        kv = torch.randn(model.stacked_kv_cache[idx][:, :, :ctx].shape, generator=gen).bfloat16()
        model.stacked_kv_cache[idx][:, :, :ctx] = kv.to(dev)
    tp = TensorParallelDecoder(model, rank, world)
    tokens = tp.decode(first, ntok, ctx)
    torch.cuda.synchronize()
    status = tp.mk.status()
    result = dict(rank=rank, tokens=tokens.cpu().tolist(), status=status["code"],
                  hidden=tp.schedule.globs.hidden_states.float().cpu().tolist(),
                  logits=tp.logits().float().cpu().tolist(),
                  k_rows=tp.local.stacked_kv_cache[0][:, 0, ctx:ctx + ntok].float().cpu().flatten().tolist())
    if rank == 0:
        # the whole model on this GPU, teacher-forced on the tokens the split model produced
        whole = MK_Generator(model, make_mk_interpreter("latency"), build_schedule(model))
        fed = [first] + result["tokens"][:-1]
        whole_tokens = []
        for i, tok in enumerate(fed):
            whole_tokens.append(int(whole.run(torch.tensor([[tok]], device=dev), pos_id=ctx + i)))
        torch.cuda.synchronize()
        g = whole.schedule.globs
        result["whole_tokens"] = whole_tokens
        result["whole_hidden"] = g.hidden_states.float().cpu().tolist()
        result["whole_logits"] = g.logits.float().cpu().tolist()
        result["whole_k_rows"] = model.stacked_kv_cache[0][:, 0, ctx:ctx + ntok].float().cpu().flatten().tolist()
    (out_dir / f"rank{rank}.json").write_text(json.dumps(result))
    dist.barrier()
    tp.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
