"""Low-latency dispatch / combine (decode batch) with one process per GPU, in CUDA graphs, with optional phase stamps.

    python benchmarks/bench_ll.py [--tokens 128 --experts 384 --phases]
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 benchmarks/bench_ll.py --phases
Prints one JSON line from rank 0: device microseconds per graph replay (maximum over ranks) and, with --phases, the
microseconds since kernel start at which block 0 of every rank finished each phase (one launch of the profile
instantiation of each kernel, outside the timed loop).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    if not torch.cuda.is_available():
        raise SystemExit("this benchmark drives the CUDA kernels and needs a GPU; bench_ep.py and bench_mega_config.py also run on the CPU engine")
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=384)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--bf16", action="store_true", help="bf16 dispatch instead of the fused fp8 quantiser")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--phases", action="store_true")
    ap.add_argument("--trace", default=None, help="with --phases: write the phase stamps of every rank as Chrome-trace / Perfetto JSON")
    args = ap.parse_args()
    from deepep_b200 import ElasticBuffer

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    T, H, E, K = args.tokens, args.hidden, args.experts, args.topk
    gen = torch.Generator().manual_seed(77 + rank)
    x = torch.randn((T, H), generator=gen).bfloat16().to(dev)
    idx = torch.stack([torch.randperm(E, generator=gen)[:K] for _ in range(T)]).to(torch.int64).to(dev)
    w = torch.softmax(torch.randn((T, K), generator=gen), dim=1).float().to(dev)
    buf = ElasticBuffer(group, num_max_tokens_per_rank=256, hidden=H, num_topk=K, use_fp8_dispatch=not args.bf16,
                        explicitly_destroy=True)

    def dispatch():
        out = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_cpu_sync=False)
        return (out[0][0] if isinstance(out[0], tuple) else out[0]), out[3]

    rx, handle = dispatch()
    assert handle.is_low_latency
    eo = torch.randn((rx.shape[0], H), device=dev).bfloat16()
    buf.combine(eo, handle)
    torch.cuda.synchronize()
    g_d, g_c = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_d):
        rx, handle = dispatch()
    with torch.cuda.graph(g_c):
        buf.combine(eo, handle)

    def timed(fn):
        for _ in range(3):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / args.iters * 1e3], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return round(t.item(), 2)

    def pair():
        g_d.replay()
        g_c.replay()

    out = dict(world=world, tokens=T, hidden=H, experts=E, topk=K, dispatch="bf16" if args.bf16 else "fp8",
               ll_dispatch_graph_us=timed(g_d.replay), ll_combine_graph_us=timed(g_c.replay), ll_roundtrip_graph_us=timed(pair))
    if args.phases:
        eng = buf.engine
        eng.enable_device_profile(True)
        for _ in range(2):          # the second launch has warm instruction caches
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            _, h2 = dispatch()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            buf.combine(eo, h2)
            torch.cuda.synchronize()
        mine = {op: {k: round(v, 1) for k, v in eng.phase_stamps(op).items()} for op in ("ll_dispatch", "ll_combine")}
        eng.enable_device_profile(False)
        gathered = [None] * world
        if world > 1:
            dist.all_gather_object(gathered, mine)
        else:
            gathered = [mine]
        out["phases_us_by_rank"] = gathered
        if args.trace and rank == 0:
            from deepep_b200.utils import trace as TR

            events = []
            for r, stamps in enumerate(gathered):
                first = TR.from_phase_stamps("ll_dispatch", stamps["ll_dispatch"], r)
                events += first + TR.from_phase_stamps("ll_combine", stamps["ll_combine"], r,
                                                       offset_us=max(list(stamps["ll_dispatch"].values()) + [0.0]))
            TR.write_trace(args.trace, events)
    if rank == 0:
        print(json.dumps(out), flush=True)
    buf.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
