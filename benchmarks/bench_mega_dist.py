"""Fused MoE layer through the public API with one process per GPU (prefill and decode batch).

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 benchmarks/bench_mega_dist.py
Prints one JSON line from rank 0: device microseconds (maximum over ranks) and whole-job tokens per second.
DEEPEP_MEGA_INTERLEAVE=0/1 selects the tile schedule (see deepep_b200/models/mega_moe.py).
"""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    if not torch.cuda.is_available():
        raise SystemExit("this benchmark drives the CUDA kernels and needs a GPU; bench_ep.py and bench_mega_config.py also run on the CPU engine")
    import bench

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD

    def timed(fn, iters):
        for _ in range(3):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / iters * 1e3], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    out = bench.bench_mega_moe(group, world, rank, dev, timed)
    out.update(world=world, interleave=os.environ.get("DEEPEP_MEGA_INTERLEAVE", "default"))
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
