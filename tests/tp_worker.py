"""Worker for tests/test_gpu_tp.py: one process per GPU (torch.distributed.run).  Runs a small Qwen3-shaped model
tensor-parallel over all ranks, with and without CUDA-graph replay, and checks on rank 0 that the greedy ids equal
the CPU oracle's and that every rank produced the same ids."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    from teenygrad_b200 import qwen3, tp
    from oracle import qwen3 as oq
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = tp.init_comm(rank, world)
    layers, hidden, hq, hkv, inter, vocab = 3, 512, 8, 8, 1024, 4096
    ocfg = oq.OracleQwen3Config(layers, hidden, hq, hkv, 128, inter, vocab, tied=False)
    sd = oq.make_weights(ocfg, 21)
    B, S, steps = 3, 40, 12
    ids = torch.randint(0, vocab, (B, S), generator=torch.Generator().manual_seed(22))
    cfg = qwen3.Qwen3Config(layers, hidden, hq, hkv, 128, inter, vocab, tied=False)
    results = []
    for graph in (False, True):
        r = qwen3.Qwen3Runner(cfg, max_batch=B, max_len=S + steps, max_new_tokens=steps, tp_rank=rank, tp_size=world,
                              comm=comm)
        r.load_state_dict(sd)
        got = r.generate(ids, steps, use_graph=graph).contiguous()
        torch.cuda.synchronize()
        assert qwen3.lib.teeny_device_error(1) == 0
        results.append(got)
        del r
    assert torch.equal(results[0], results[1]), "graph replay differs from eager under tensor parallelism"
    gathered = [torch.empty_like(results[0]) for _ in range(world)]
    dist.all_gather(gathered, results[0])
    if rank == 0:
        for g in gathered:
            assert torch.equal(g, gathered[0]), "ranks disagree on the generated ids"
        want = oq.OracleQwen3(ocfg, sd).generate(ids, steps)
        assert torch.equal(gathered[0].cpu().long(), want), (gathered[0].cpu(), want)
        print(f"TP{world} OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
