"""alltoallv_gmm / gmm_alltoallv timing against an NCCL all-to-all-v + cuBLAS baseline.

One GPU (virtual ranks share the device; the baseline is the grouped matmul alone, without a transfer):
    python benchmarks/bench_gmm.py --world 1 --rows 32768 --in-features 7168 --out-features 4096 --experts 4
Several GPUs, one process each (public API; the baseline is all_to_all_single + one matmul per expert):
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_gmm.py --rows 32768 --experts 32
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def timed(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters * 1e3


def even_counts(rows, experts):
    base = rows // experts
    c = [base] * experts
    c[-1] += rows - base * experts
    return c


def virtual(args):
    from deepep_b200.ops import ep_gmm_fused as G
    from deepep_b200.ops import load_native

    C = load_native()
    dev = torch.device("cuda")
    P, R, K, N, E = args.world, args.rows, args.k, args.n, args.experts
    L = E // P
    layout = C.make_mega_layout(P, 1, 128, 1, G.GmmEngine.region_bytes(C, R, max(K, N), max(K, N)))
    sessions = [C.Session(r, P, layout.total, 30.0) for r in range(P)]
    for s in sessions:
        s.attach_peers([q.workspace for q in sessions])
    eng = G.GmmEngine(sessions, layout, dev, R, max(K, N), max(K, N))
    counts = even_counts(R, E)
    d_c = [torch.tensor(counts, dtype=torch.int32, device=dev) for _ in range(P)]
    xs = [torch.randn((R, K), device=dev).to(torch.bfloat16) for _ in range(P)]
    w1 = [(torch.randn((L, K, N), device=dev) / K ** 0.5).to(torch.bfloat16) for _ in range(P)]
    w2 = [(torch.randn((L, N, K), device=dev) / N ** 0.5).to(torch.bfloat16) for _ in range(P)]
    recv = sum(counts[r * L:(r + 1) * L][l] for r in range(1) for l in range(L)) * P     # even routing: same on every rank
    outs = [torch.empty((recv, N), dtype=torch.bfloat16, device=dev) for _ in range(P)]
    back = [torch.empty((R, K), dtype=torch.bfloat16, device=dev) for _ in range(P)]
    t1 = timed(lambda: eng.a2av_gmm(xs, w1, d_c, outs, num_experts=E), args.iters)
    t2 = timed(lambda: eng.gmm_a2av(outs, w2, d_c, back, num_experts=E), args.iters)
    # zero-copy variants: x lives in the stage area, the returned rows stay in the receive area
    sx = [eng.symmetric_input(r, R, K) for r in range(P)]
    for r in range(P):
        sx[r].copy_(xs[r])
    so = [eng.symmetric_output(r, R, K) for r in range(P)]
    t1z = timed(lambda: eng.a2av_gmm(sx, w1, d_c, outs, num_experts=E), args.iters)
    t2z = timed(lambda: eng.gmm_a2av(outs, w2, d_c, so, num_experts=E), args.iters)
    eng.check()
    per = recv // L

    def cublas():
        for l in range(L):
            torch.matmul(xs[0][l * per:(l + 1) * per], w1[0][l], out=outs[0][l * per:(l + 1) * per])
    tb = timed(cublas, args.iters) if P == 1 else None
    flops = 2.0 * P * recv * K * N
    print(json.dumps({"mode": "virtual", "world": P, "rows": R, "k": K, "n": N, "experts": E,
                      "a2av_gmm_us": t1, "a2av_gmm_zero_copy_us": t1z, "gmm_a2av_zero_copy_us": t2z, "a2av_gmm_tflops": flops / t1 / 1e6, "gmm_a2av_us": t2, "gmm_a2av_tflops": flops / t2 / 1e6,
                      "cublas_gmm_only_us": tb, "cublas_tflops": flops / tb / 1e6 if tb else None}))
    for s in sessions:
        s.close()


def distributed(args):
    import torch.distributed as dist

    from deepep_b200.ops import ep_gmm_fused as G

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    dev = torch.device("cuda")
    R, K, N, E = args.rows, args.k, args.n, args.experts
    L = E // world
    G.init_group(dist.group.WORLD, max_rows=R, max_k=max(K, N), max_n=max(K, N))
    counts = even_counts(R, E)
    glob = [counts[rank * L + l] for _ in range(world) for l in range(L)]
    recv = sum(glob)
    d_local = torch.tensor(counts, dtype=torch.int32, device=dev)
    d_glob = torch.tensor(glob, dtype=torch.int32, device=dev)
    x = torch.randn((R, K), device=dev).to(torch.bfloat16)
    w1 = (torch.randn((L, K, N), device=dev) / K ** 0.5).to(torch.bfloat16)
    w2 = (torch.randn((L, N, K), device=dev) / N ** 0.5).to(torch.bfloat16)
    out = torch.empty((recv, N), dtype=torch.bfloat16, device=dev)
    back = torch.empty((R, K), dtype=torch.bfloat16, device=dev)

    def fused1():
        G.alltoallv_gmm(x, w1, d_local, d_glob, ep_size=world, expert_num=E, received_rows=recv, out=out)

    def fused2():
        G.gmm_alltoallv(out, w2, d_local, d_glob, ep_size=world, expert_num=E, out=back)

    # baseline: NCCL all-to-all-v (rows are already grouped by destination rank) + one cuBLAS matmul per expert
    send_split = [sum(counts[d * L:(d + 1) * L]) for d in range(world)]
    recv_split = [sum(counts[rank * L:(rank + 1) * L])] * world
    gathered = torch.empty((recv, K), dtype=torch.bfloat16, device=dev)
    order = torch.arange(recv, device=dev).view(world, L, -1).transpose(0, 1).reshape(-1)   # (source, expert) -> (expert, source)
    per = recv // L
    ret = torch.empty((recv, K), dtype=torch.bfloat16, device=dev)

    def base1():
        dist.all_to_all_single(gathered, x, recv_split, send_split)
        a = gathered[order] if recv % (world * L) == 0 else gathered
        for l in range(L):
            torch.matmul(a[l * per:(l + 1) * per], w1[l], out=out[l * per:(l + 1) * per])

    def base2():
        for l in range(L):
            torch.matmul(out[l * per:(l + 1) * per], w2[l], out=ret[l * per:(l + 1) * per])
        dist.all_to_all_single(back, ret, send_split, recv_split)

    res = {}
    for name, fn in (("a2av_gmm", fused1), ("gmm_a2av", fused2), ("nccl_cublas_a2av_gmm", base1), ("nccl_cublas_gmm_a2av", base2)):
        dist.barrier()
        t = torch.tensor([timed(fn, args.iters)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[name + "_us"] = t.item()
    flops = 2.0 * recv * K * N
    link_bytes = R * (world - 1) / world * K * 2
    if rank == 0:
        res.update(mode="distributed", world=world, rows=R, k=K, n=N, experts=E,
                   a2av_gmm_tflops_per_gpu=flops / res["a2av_gmm_us"] / 1e6, gmm_a2av_tflops_per_gpu=flops / res["gmm_a2av_us"] / 1e6,
                   a2av_nvlink_gbs=link_bytes / res["a2av_gmm_us"] / 1e3,
                   speedup_a2av_gmm=res["nccl_cublas_a2av_gmm_us"] / res["a2av_gmm_us"],
                   speedup_gmm_a2av=res["nccl_cublas_gmm_a2av_us"] / res["gmm_a2av_us"])
        print(json.dumps(res))
    G.destroy_group()
    dist.destroy_process_group()


if __name__ == "__main__":
    if not torch.cuda.is_available():
        raise SystemExit("this benchmark drives the CUDA kernels and needs a GPU; bench_ep.py and bench_mega_config.py also run on the CPU engine")
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=1, help="virtual ranks on one GPU (ignored under torchrun)")
    ap.add_argument("--rows", type=int, default=32768, help="rows per rank (tokens x top-k)")
    ap.add_argument("--in-features", dest="k", type=int, default=7168)
    ap.add_argument("--out-features", dest="n", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=4)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    distributed(a) if "WORLD_SIZE" in os.environ and int(os.environ["WORLD_SIZE"]) > 1 else virtual(a)
