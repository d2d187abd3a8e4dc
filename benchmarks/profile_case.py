"""One small notify -> dispatch -> combine pass with N virtual ranks on one GPU, for profiler captures.

    python benchmarks/profile_case.py --world 1 --tokens 1024 --repeat 2
"""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--repeat", type=int, default=2)
    ap.add_argument("--blocks", type=int, default=0)
    ap.add_argument("--mode", type=int, default=0, help="0 bf16, 2 fused fp8")
    args = ap.parse_args()
    from deepep_b200.parallel.virtual import VirtualWorld
    from helpers import group_limited_routes

    dev = torch.device("cuda")
    P, T, H, E, K = args.world, args.tokens, args.hidden, args.experts, args.topk
    xs = [torch.randn((T, H), device=dev, dtype=torch.bfloat16) for _ in range(P)]
    idx = [group_limited_routes(T, E, K, 8, 4, seed=r).to(dev) for r in range(P)]
    with VirtualWorld(P, T, H, K, timeout=20.0) as vw:
        eng = vw.engine
        for _ in range(args.repeat):
            plans = eng.notify(idx, [None] * P, E)
            outs = eng.dispatch(xs, plans, args.mode, blocks=args.blocks)
            if args.mode == 0:
                eng.combine([o[0] for o in outs], plans, [None] * P, blocks=args.blocks)
        torch.cuda.synchronize()
        eng.check_status()
    print("done")


if __name__ == "__main__":
    main()
