"""Sweep of SM budgets for the high-throughput dispatch/combine and timing of notify and the low-latency pair.

One process per GPU (launch with torch.distributed.run) or a single process:
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/sweep_ht.py --blocks 48 64 96 128
Prints one JSON line per configuration (device time, maximum over ranks).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--blocks", type=int, nargs="+", default=[64, 96, 128])
    ap.add_argument("--send-frac", type=float, nargs="+", default=[0.3, 0.5])
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--ll", action="store_true")
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--remote-only", action="store_true", help="route every token only to experts of the next rank (link stress)")
    args = ap.parse_args()
    from deepep_b200 import ElasticBuffer
    from helpers import group_limited_routes

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    T, H, E, K = args.tokens, args.hidden, 256, args.topk
    x = torch.randn((T, H), device=dev).bfloat16()
    if args.remote_only:
        local_e = E // world
        base = ((rank + 1) % world) * local_e
        idx = (base + torch.stack([torch.randperm(local_e, device=dev)[:K] for _ in range(T)])).to(torch.int64)
    else:
        idx = group_limited_routes(T, E, K, 8, 4, seed=rank).to(dev)
    w = torch.softmax(torch.randn((T, K), device=dev), dim=1)
    buf = ElasticBuffer(group, num_max_tokens_per_rank=T, hidden=H, num_topk=K, explicitly_destroy=True)
    eng = buf.engine

    def timed(fn, iters):
        for _ in range(2):
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
        return float(t.item())

    def say(**kw):
        if rank == 0:
            print(json.dumps(kw), flush=True)

    plan = eng.notify([idx], [w], E)[0]
    say(op="notify+sync", us=timed(lambda: eng.notify([idx], [w], E), args.iters))
    say(op="notify_kernel", us=timed(lambda: eng.notify([idx], [w], E, cpu_sync=False), args.iters))
    rows = eng.dispatch([x], [plan], 0)[0][0]
    for blocks in args.blocks:
        for frac in args.send_frac:
            def disp():
                send, recv = eng.split_blocks(blocks, frac)
                eng.C.dispatch(eng.layout, eng.sessions, [disp_args], send, recv, torch.cuda.current_stream().cuda_stream)
            recv_x = torch.empty_like(rows)
            disp_args = dict(x=x.data_ptr(), x_sf=None, T=T, mode=0, send_slot=plan.send_slot.data_ptr(),
                             stage_meta=plan.stage_meta.data_ptr(), chunk_start=plan.chunk_start.data_ptr(),
                             rank_tokens=plan.rank_tokens.data_ptr(), meta_stride=plan.meta_stride, recv_x=recv_x.data_ptr(), recv_sf=None)
            say(op="dispatch_bf16", blocks=blocks, send_frac=frac, us=timed(disp, args.iters))
            out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
            comb_args = dict(x=rows.data_ptr(), w=None, stage_meta=plan.stage_meta.data_ptr(), chunk_start=plan.chunk_start.data_ptr(),
                             rank_tokens=plan.rank_tokens.data_ptr(), send_slot=plan.send_slot.data_ptr(), topk_idx=idx.data_ptr(),
                             T=T, meta_stride=plan.meta_stride, K=K, E=E, expand=1, bias0=None, bias1=None, out=out.data_ptr(), out_w=None)

            def comb():
                send, recv = eng.split_blocks(blocks, 1.0 - frac)
                eng.C.combine(eng.layout, eng.sessions, [comb_args], send, recv, torch.cuda.current_stream().cuda_stream)
            say(op="combine_bf16", blocks=blocks, expert_frac=1.0 - frac, us=timed(comb, args.iters))
    buf.destroy()
    if args.ll:
        Tl, El = 128, 384
        xl = torch.randn((Tl, H), device=dev).bfloat16()
        il = torch.stack([torch.randperm(El, device=dev)[:K] for _ in range(Tl)]).to(torch.int64)
        wl = torch.softmax(torch.randn((Tl, K), device=dev), dim=1)
        b2 = ElasticBuffer(group, num_max_tokens_per_rank=256, hidden=H, num_topk=K, use_fp8_dispatch=True, explicitly_destroy=True)
        (rx, rsf), _, rw, h, _ = b2.dispatch(xl, topk_idx=il, topk_weights=wl, num_experts=El, do_cpu_sync=False)
        eo = torch.randn((rx.shape[0], H), device=dev).bfloat16()
        say(op="ll_dispatch_fp8", us=timed(lambda: b2.dispatch(xl, topk_idx=il, topk_weights=wl, num_experts=El, do_cpu_sync=False), 10))
        say(op="ll_combine", us=timed(lambda: b2.combine(eo, h), 10))
        b2.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
