"""Fused MoE layer from a model configuration in the reference's schema, through the public API.

    python benchmarks/bench_mega_config.py --config benchmarks/configs/mega_smoke.json --check
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_mega_config.py \
        --config benchmarks/configs/mega_deepseek_v4_pro.json
The configuration names the model (hidden, intermediate size, experts, top-k, shared experts per rank) and the batch
sizes per rank (``deepep_b200.models.mega_tools.load_model_config``; the reference ships the same files with its
megamoe package).  Every rank holds ``experts / world`` routed experts and its own shared experts, draws a batch of each
size, and runs ``fp8_fp4_mega_moe``.  Rank 0 prints one JSON line: per batch size the time of the slowest rank
(CUDA events on a GPU, the host clock on the CPU engine), whole-job tokens per second and TFLOP/s per rank.
``--check`` (one rank only, small models) compares the output with the fp32 restatement of the layer.
Without a GPU the layer runs on the CPU engine and the ranks meet through the launcher's TCPStore.
"""
import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def expert_weights(count, H, I, seed, dev):
    """``count`` experts of random e2m1 weights with ue8m0 scales around 2^(-log2(K)/2 - 3), generated on ``dev``."""
    g = torch.Generator(device=dev).manual_seed(seed)
    out = []
    for n, k in ((2 * I, H), (H, I)):
        packed = torch.randint(0, 256, (count, n, k // 2), dtype=torch.uint8, device=dev, generator=g)
        centre = 127 + int(-0.5 * torch.log2(torch.tensor(float(k))).item()) - 3
        scales = torch.randint(centre - 1, centre + 2, (count, n, k // 32), dtype=torch.uint8, device=dev, generator=g)
        out.append((packed, scales))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--check", action="store_true", help="compare with the fp32 restatement (one rank, small models)")
    args = ap.parse_args()
    from deepep_b200.models import mega_tools as MT
    from deepep_b200.models.mega_moe import SymmBuffer, fp8_fp4_mega_moe, transform_weights_for_mega_moe
    from deepep_b200.oracle import megamoe as O
    from deepep_b200.utils.math import per_token_cast_to_fp8

    cfg = MT.load_model_config(args.config)
    m = cfg["model"]
    H, I, E, K, S = m["hidden"], m["intermediate_hidden"], m["num_experts"], m["num_topk"], m["num_shared_experts"]
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if E % world:
        raise SystemExit(f"{E} experts do not divide over {world} ranks")
    cuda = torch.cuda.is_available()
    group = None
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
        if world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=dev)
            group = dist.group.WORLD
    else:
        dev = torch.device("cpu")
    L = E // world
    l1, l2 = expert_weights(L, H, I, cfg["seed"] + 1000 * rank, dev)
    w1, w2 = transform_weights_for_mega_moe(l1, l2, device=dev)
    shared = None
    if S:
        s1, s2 = expert_weights(S, H, I, cfg["seed"] + 1000 * rank + 500, dev)
        shared = (s1, s2) + transform_weights_for_mega_moe(s1, s2, device=dev)
    cap = max(cfg["bs_values"])
    where = dict(rank=rank, world_size=world) if (group is None and world > 1) else {}
    buf = SymmBuffer(group, E, cap, K, H, I, num_shared_experts=S, **where)
    sync = (lambda: torch.cuda.synchronize(dev)) if cuda else (lambda: None)
    rows = []
    for bs in cfg["bs_values"]:
        g = torch.Generator().manual_seed(cfg["seed"] + 7 * rank + bs)
        x = torch.randn((bs, H), generator=g).bfloat16().to(dev)
        idx = torch.rand((bs, E), generator=g).topk(K, dim=1).indices.to(dev)
        w = torch.softmax(torch.randn((bs, K), generator=g), dim=1).to(dev)
        q, sf = per_token_cast_to_fp8(x, use_ue8m0=True)
        buf.load_inputs(q, sf, idx, w)
        y = torch.empty((bs, H), dtype=torch.bfloat16, device=dev)
        run = (lambda: fp8_fp4_mega_moe(y, w1, w2, buf, shared[2], shared[3])) if shared else (lambda: fp8_fp4_mega_moe(y, w1, w2, buf))
        run()
        sync()
        buf.engine.check()
        row = dict(bs=bs)
        if args.check:
            if world != 1:
                raise SystemExit("--check needs all experts on one rank")
            O.FP4_VALUES = O.FP4_VALUES.to(dev)
            codes = buf.x_sf[:bs]
            golden = O.mega_moe_reference([(q, codes)], [idx], [w], l1, l2, E, shared[0] if shared else None,
                                          shared[1] if shared else None)[0]
            verdict = MT.compare(y, golden)
            row.update(ok=bool(verdict["ok"]), mare=verdict["mare"])
        for _ in range(cfg["warmup"]):
            run()
        buf.control.barrier()
        sync()
        if cuda:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(cfg["iters"]):
                run()
            end.record()
            sync()
            us = start.elapsed_time(end) * 1e3 / cfg["iters"]
        else:
            t0 = time.perf_counter()
            for _ in range(cfg["iters"]):
                run()
            us = (time.perf_counter() - t0) * 1e6 / cfg["iters"]
        us = max(buf.control.all_gather_object(float(us)))
        routed = bs * (K + S)                         # rows a rank's experts see when the routing is even
        row.update(us=round(us, 1), tokens_per_s=round(world * bs / (us * 1e-6)), tflops_per_rank=round(6.0 * routed * H * I / (us * 1e-6) / 1e12, 2))
        rows.append(row)
    buf.destroy()
    if rank == 0:
        print(json.dumps(dict(config=os.path.basename(args.config), model=m, world=world, engine="cuda" if cuda else "cpu",
                              iters=cfg["iters"], results=rows)), flush=True)
    if group is not None:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0 if all(r.get("ok", True) for r in rows) else 1


if __name__ == "__main__":
    sys.exit(main())
