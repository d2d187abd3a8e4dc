"""Fused MoE forward timing on one GPU (N virtual ranks share the device) with a per-kernel breakdown.

    python benchmarks/bench_mega.py --world 1 --tokens 4096 --experts 32      # one rank's share of an EP8 layer
    python benchmarks/bench_mega.py --accuracy --world 2 --tokens 256 --hidden 1024 --inter 512 --experts 8
                                                  # MARE / MERE / RMSE and the mixed-error gate against the cached CPU golden
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
    ap.add_argument("--world", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--unfused", action="store_true", help="four launches instead of the persistent kernel")
    ap.add_argument("--accuracy", action="store_true", help="compare with the CPU golden instead of timing")
    ap.add_argument("--golden-dir", default=os.path.join(ROOT, "benchmarks", ".golden_cache"))
    ap.add_argument("--no-profiler", action="store_true", help="skip the torch.profiler breakdown (needed under ncu)")
    ap.add_argument("--pairs", choices=["auto", "0", "1"], default=None, help="CTA pairs in the fused kernel (default: the engine's rule)")
    ap.add_argument("--phases", action="store_true", help="one extra launch with the per-CTA phase timer; prints the breakdown")
    ap.add_argument("--trace", default=None, help="with --phases: write the per-CTA phase spans as Chrome-trace / Perfetto JSON")
    args = ap.parse_args()
    from deepep_b200.models.mega_moe import MegaEngine, MegaWeights
    from deepep_b200.ops import load_native

    C = load_native()
    dev = torch.device("cuda")
    P, T, H, I, E, K = args.world, args.tokens, args.hidden, args.inter, args.experts, args.topk
    if args.accuracy:
        return accuracy(args, C, dev)
    L = E // P
    layout = C.make_mega_layout(P, T, H, K, MegaEngine.mega_bytes(C, T, H, K))
    sessions = [C.Session(r, P, layout.total, 30.0) for r in range(P)]
    for s in sessions:
        s.attach_peers([q.workspace for q in sessions])
    eng = MegaEngine(sessions, layout, dev, E, I)
    if args.pairs is not None:
        eng.pairs = args.pairs
    g = torch.Generator(device="cuda").manual_seed(0)
    w1 = [MegaWeights(torch.randint(0, 256, (L * 2 * I * (H // 128), 64), dtype=torch.uint8, device=dev, generator=g),
                      torch.full((L * 2 * I // 128 * (H // 128) * 512,), 118, dtype=torch.uint8, device=dev), L, 2 * I, H) for _ in range(P)]
    w2 = [MegaWeights(torch.randint(0, 256, (L * H * (I // 128), 64), dtype=torch.uint8, device=dev, generator=g),
                      torch.full((L * H // 128 * (I // 128) * 512,), 120, dtype=torch.uint8, device=dev), L, H, I) for _ in range(P)]
    for r in range(P):
        x, sf, ti, tw = eng.input_views(r)
        x.view(torch.uint8).copy_(torch.randint(0, 120, (T, H), dtype=torch.uint8, device=dev, generator=g))
        sf.fill_(127)
        scores = torch.rand((T, E), device=dev, generator=g)
        ti.copy_(torch.topk(scores, K, dim=1).indices.to(torch.int32))
        tw.copy_(torch.softmax(torch.randn((T, K), device=dev, generator=g), dim=1))
    ys = [torch.empty((T, H), dtype=torch.bfloat16, device=dev) for _ in range(P)]

    def run():
        eng.forward(ys, [T] * P, w1, w2, fused=not args.unfused)

    for _ in range(2):
        run()
    torch.cuda.synchronize()
    eng.check()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.iters):
        run()
    e.record()
    torch.cuda.synchronize()
    total_us = s.elapsed_time(e) / args.iters * 1e3
    # per-kernel breakdown from the profiler (device time)
    kern = {}
    if not args.no_profiler:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            run()
            torch.cuda.synchronize()
        for evt in prof.events():
            if evt.device_time > 0:
                kern.setdefault(evt.name.split("(")[0][-40:], []).append(evt.device_time)
    phases = None
    if args.phases and not args.unfused:
        from deepep_b200.models.mega_tools import parse_timer

        timer = torch.zeros((eng.sm_count, C.mega_timer_words), dtype=torch.int64, device=dev)
        eng.forward(ys, [T] * P, w1, w2, fused=True, timer=timer)
        torch.cuda.synchronize()
        phases = {k: round(v, 1) if isinstance(v, float) else v for k, v in parse_timer(timer).items()}
        if args.trace:
            from deepep_b200.utils import trace as TR

            TR.write_trace(args.trace, TR.from_mega_timer(timer))
    rows = P * T * K
    flops = 2.0 * rows * (2 * I) * H + 2.0 * rows * H * I
    print(json.dumps({"world": P, "tokens": T, "hidden": H, "inter": I, "experts": E, "topk": K, "total_us": total_us,
                      "tokens_per_s": P * T / (total_us * 1e-6), "tflops": flops / (total_us * 1e-6) / 1e12, "cta_pairs": bool(eng.use_pairs([T] * P)) and not args.unfused,
                      "kernels_us": {k: v for k, v in kern.items()}, **({"phases_us": phases} if phases else {})}))
    torch.cuda.synchronize()
    for s_ in sessions:
        s_.close()


def accuracy(args, C, dev):
    from deepep_b200.models import mega_tools as tools
    from deepep_b200.models.mega_moe import MegaEngine, transform_weights_for_mega_moe

    P, T, H, I, E, K = args.world, args.tokens, args.hidden, args.inter, args.experts, args.topk
    L = E // P
    spec = tools.contract(world=P, tokens=[T] * P, hidden=H, intermediate=I, experts=E, topk=K, seed=0)
    xs, idx, ws, l1, l2 = tools.make_case(spec)
    for r in range(P):
        tools.check_routing(idx[r].tolist(), ws[r].tolist(), E, K)
    layout = C.make_mega_layout(P, T, H, K, MegaEngine.mega_bytes(C, T, H, K))
    sessions = [C.Session(r, P, layout.total, 30.0) for r in range(P)]
    for s in sessions:
        s.attach_peers([q.workspace for q in sessions])
    eng = MegaEngine(sessions, layout, dev, E, I)
    w = [transform_weights_for_mega_moe((l1[0][r * L:(r + 1) * L], l1[1][r * L:(r + 1) * L]),
                                        (l2[0][r * L:(r + 1) * L], l2[1][r * L:(r + 1) * L]), device=dev) for r in range(P)]
    for r in range(P):
        x, sf, ti, tw = eng.input_views(r)
        x[:T].copy_(xs[r][0]); sf[:T].copy_(xs[r][1]); ti[:T].copy_(idx[r].to(torch.int32)); tw[:T].copy_(ws[r])
    ys = [torch.zeros((T, H), dtype=torch.bfloat16, device=dev) for _ in range(P)]
    eng.forward(ys, [T] * P, [a for a, _ in w], [b for _, b in w], fused=not args.unfused)
    torch.cuda.synchronize()
    eng.check()
    ok, rows = tools.accuracy_report(ys, spec, args.golden_dir)
    print(json.dumps({"accuracy_ok": ok, "spec": spec, "ranks": rows}))
    for s in sessions:
        s.close()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main() or 0)
