"""One low-latency dispatch + combine pass (decode shape) with N virtual ranks on one GPU, for profiler captures.

    python benchmarks/profile_ll.py --world 1 --repeat 3
"""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=384)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--repeat", type=int, default=3)
    args = ap.parse_args()
    from deepep_b200.ops import load_native
    from deepep_b200.parallel.virtual import VirtualWorld

    C = load_native()
    dev = torch.device("cuda")
    P, T, H, E, K, M = args.world, args.tokens, args.hidden, args.experts, args.topk, 256
    with VirtualWorld(P, M, H, K, timeout=10.0, ll_bytes=C.ll_region_bytes(P, M, K, H)) as vw:
        eng = vw.engine
        xs = [torch.randn((T, H), device=dev).bfloat16() for _ in range(P)]
        idx = [torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(T)]).to(torch.int64) for _ in range(P)]
        ws = [torch.softmax(torch.randn((T, K), device=dev), 1) for _ in range(P)]
        for _ in range(args.repeat):
            res = eng.ll_dispatch(xs, idx, ws, E, 2, cpu_sync=False)
            plans = [r[0] for r in res]
            eng.ll_combine([torch.zeros((p.num_rows, H), device=dev, dtype=torch.bfloat16) for p in plans], plans)
        torch.cuda.synchronize()
        eng.check_status()
    print("done")


if __name__ == "__main__":
    main()
