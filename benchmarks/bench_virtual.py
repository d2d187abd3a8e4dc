"""Single-GPU benchmark of the high-throughput kernels with N virtual ranks on one device.

All N ranks run inside one cooperative launch and share the GPU's SMs and HBM, so the numbers
measure how close the copy/reduce machinery gets to the HBM roofline (there is no NVLink in
this setting): ``python benchmarks/bench_virtual.py --world 8 --tokens 4096``.
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    if not torch.cuda.is_available():
        raise SystemExit("this benchmark drives the CUDA kernels and needs a GPU; bench_ep.py and bench_mega_config.py also run on the CPU engine")
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--blocks", type=int, default=0)
    ap.add_argument("--fp8", action="store_true")
    args = ap.parse_args()
    from deepep_b200.parallel.virtual import VirtualWorld
    from deepep_b200.utils.routing import group_limited_routes

    dev = torch.device("cuda")
    P, T, H, E, K = args.world, args.tokens, args.hidden, args.experts, args.topk
    xs = [torch.randn((T, H), device=dev, dtype=torch.bfloat16) for _ in range(P)]
    idx = [group_limited_routes(T, E, K, 8, 4, seed=r).to(dev) for r in range(P)]
    with VirtualWorld(P, T, H, K, timeout=20.0) as vw:
        eng = vw.engine
        plans = eng.notify(idx, [None] * P, E)
        mode = 2 if args.fp8 else 0

        def timed(fn):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(args.iters):
                fn()
            e.record()
            torch.cuda.synchronize()
            eng.check_status()
            return s.elapsed_time(e) / args.iters * 1e3

        t_notify = timed(lambda: eng.notify(idx, [None] * P, E))
        t_disp = timed(lambda: eng.dispatch(xs, plans, mode, blocks=args.blocks))
        outs = eng.dispatch(xs, plans, 0, blocks=args.blocks)
        eo = [o[0] for o in outs]
        t_comb = timed(lambda: eng.combine(eo, plans, [None] * P, blocks=args.blocks))
        rows = sum(p.num_rows for p in plans)
        staged = sum(p.num_staged_rows for p in plans)
        row_b = H * 2
        hbm_disp = (P * T + staged) * row_b + staged * row_b + rows * row_b      # read x, write+read staging, write rows
        hbm_comb = rows * row_b + staged * row_b * 2 + P * T * row_b             # read rows, write+read partials, write out
        print(json.dumps({"world": P, "tokens": T, "hidden": H, "rows": rows, "staged_rows": staged,
                          "notify_us": t_notify, "dispatch_us": t_disp, "combine_us": t_comb,
                          "dispatch_hbm_GBps": hbm_disp / t_disp / 1e3, "combine_hbm_GBps": hbm_comb / t_comb / 1e3}))


if __name__ == "__main__":
    main()
