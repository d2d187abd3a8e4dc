"""Config-driven dispatch / combine / round-trip benchmark with versioned result records.

    python benchmarks/bench_ep.py --config benchmarks/configs/smoke.json
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_ep.py \
        --config benchmarks/configs/prefill_bf16.json --results-dir benchmarks/results
Every rank times each iteration with CUDA events (host clock on the CPU engine); rank 0 gathers the samples, takes
the per-iteration maximum over ranks and prints one JSON record (schema in deepep_b200/utils/workload.py).  The
outputs of the first iteration are compared with the all-rank CPU oracle unless --no-check is given.
``--set name=value`` changes a field of the configuration, ``--matrix name=[v1,v2]`` runs every combination of the listed
values as cases of their own (one record each), ``--dry-run`` prints the validated plan without measuring,
``--csv FILE`` appends a one-row summary (with ``--baseline-us`` a speed-up column).

``--sweep-blocks B... --sweep-fractions F...`` additionally times the cached dispatch and the combine of the same
workload for every (blocks per rank, share of the blocks on the NVLink side) pair and prints one JSON line each
(device time, maximum over ranks, and the NVLink bytes one rank sends per second); ``--device-profile`` adds the
per-block records of the kernels' profile instantiation for the default split.
"""
import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--results-dir", default=None, help="write the record there (existing files are never overwritten)")
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--set", dest="overrides", action="append", default=[], metavar="NAME=VALUE",
                    help="change one field of the configuration (JSON value), e.g. --set iterations=50 --set route=skew")
    ap.add_argument("--matrix", action="append", default=[], metavar="NAME=[V1,V2,...]",
                    help="run one case per value (several --matrix flags: every combination), one record per case")
    ap.add_argument("--dry-run", action="store_true", help="validate, print the planned record and stop: nothing is measured")
    ap.add_argument("--csv", default=None, help="rank 0 appends the record's summary row to this CSV file")
    ap.add_argument("--baseline-us", type=float, default=None, help="latency measured elsewhere for this configuration; "
                                                                   "fills the CSV's baseline and speed-up columns")
    ap.add_argument("--sweep-blocks", type=int, nargs="*", default=[], help="blocks (SMs) per rank to try")
    ap.add_argument("--sweep-fractions", type=float, nargs="*", default=[0.3, 0.4, 0.5, 0.6],
                    help="share of the blocks that drives NVLink (dispatch senders / combine expert side)")
    ap.add_argument("--device-profile", action="store_true", help="per-block records of the profile kernels (CUDA engine)")
    ap.add_argument("--trace", default=None, help="with --device-profile: write the records of every rank as Chrome-trace / "
                                                  "Perfetto JSON to this path (rank 0 writes)")
    args = ap.parse_args()

    from deepep_b200 import ElasticBuffer
    from deepep_b200.oracle import reference as R
    from deepep_b200.utils import workload as W
    from deepep_b200.utils.testing import flush_l2_cache

    cases = W.expand_matrix(W.with_overrides(W.WorkloadConfig.from_json(args.config), args.overrides), args.matrix)
    if args.dry_run:              # no framework state, no device: a plan carries the configuration and its fingerprint only
        planned = [W.plan(cfg) for cfg in cases]
        for one in planned:
            print(json.dumps(one))
        if args.results_dir:
            os.makedirs(args.results_dir, exist_ok=True)
            with open(os.path.join(args.results_dir, "plan.json"), "x") as f:
                json.dump(planned[0] if len(planned) == 1 else planned, f, indent=1, sort_keys=True)
        return 0
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if any(world != cfg.world_size for cfg in cases):
        raise SystemExit(f"the configuration is for {cases[0].world_size} ranks, this job has {world}")
    cuda = torch.cuda.is_available()
    group = None
    if world > 1:
        import torch.distributed as dist

        if cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dist.init_process_group("nccl" if cuda else "gloo")
        group = dist.group.WORLD
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")

    def run_case(cfg):
        routes = [W.make_routes(cfg, r) for r in range(world)]           # every rank can rebuild all inputs (oracle, traffic)
        xs = [torch.randn((cfg.tokens_per_rank[r], cfg.hidden), generator=torch.Generator().manual_seed(cfg.seed + 77 * r)).bfloat16()
              for r in range(world)]
        x, idx, w = xs[rank].to(dev), routes[rank][0].to(dev), (routes[rank][1].to(dev) if cfg.with_weights else None)
        expand = cfg.layout == "expanded"
        buf = ElasticBuffer(group, num_max_tokens_per_rank=max(max(cfg.tokens_per_rank), 257), hidden=cfg.hidden, num_topk=cfg.topk,
                            use_fp8_dispatch=cfg.dtype == "fp8", explicitly_destroy=True)

        def fresh():
            return buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=cfg.experts, do_expand=expand,
                                expert_alignment=cfg.alignment)

        recv, _, recv_w, handle, _ = fresh()
        rows = recv[0] if isinstance(recv, tuple) else recv
        back = torch.randn(rows.shape, device=dev).bfloat16() if cfg.dtype == "fp8" else rows

        correctness = "not_run"
        if not args.no_check:
            ref, lays = R.dispatch(xs, [r[0] for r in routes], [r[1] for r in routes] if cfg.with_weights else None, cfg.experts,
                                   do_expand=expand, expert_alignment=cfg.alignment)
            good = True
            if cfg.dtype == "bf16":
                good = torch.equal(rows.cpu().view(torch.int16), ref[rank][0].view(torch.int16))
                out = buf.combine(rows, handle)[0]
                cref = R.combine([r[0] for r in ref], lays, list(cfg.tokens_per_rank), cfg.topk)
                good = good and torch.equal(out.cpu().view(torch.int16), cref[rank][0].view(torch.int16))
            else:
                good = rows.shape[0] == ref[rank][0].shape[0]
            verdicts = buf.control.all_gather_object(bool(good)) if world > 1 else [good]
            correctness = "passed" if all(verdicts) else "failed"

        ops = {"dispatch": (fresh if cfg.dispatch_mode == "fresh" else (lambda: buf.dispatch(x, handle=handle))),
               "combine": lambda: buf.combine(back, handle)}

        def roundtrip():
            r, _, _, h, _ = fresh() if cfg.dispatch_mode == "fresh" else buf.dispatch(x, handle=handle)
            rr = r[0] if isinstance(r, tuple) else r
            buf.combine(back if cfg.dtype == "fp8" else rr, h)
        ops["roundtrip"] = roundtrip
        fn = ops[cfg.operation]

        samples = []
        for it in range(cfg.warmup + cfg.iterations):
            buf.barrier()
            if cuda:
                flush_l2_cache()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                fn()
                e.record()
                e.synchronize()
                us = s.elapsed_time(e) * 1e3
            else:
                t0 = time.perf_counter_ns()
                fn()
                us = (time.perf_counter_ns() - t0) / 1e3
            if it >= cfg.warmup:
                samples.append(max(us, 1e-3))
        if cuda and (args.sweep_blocks or args.device_profile):
            sweep(buf, cfg, x, handle, back, routes, rank, world, args, fresh)
        gathered = buf.control.all_gather_object(samples) if world > 1 else [samples]
        record = W.complete(W.plan(cfg), gathered, W.traffic(cfg, [r[0] for r in routes])["effective_bytes"], correctness)
        record["engine"] = "cuda" if cuda else "cpu"
        buf.destroy()
        if rank == 0:
            slim = {k: v for k, v in record.items() if k != "rank_samples_us"}
            print(json.dumps(slim))
            if args.results_dir:
                print("written:", W.write_result(args.results_dir, record), file=sys.stderr)
            if args.csv:
                new = not os.path.exists(args.csv) or os.path.getsize(args.csv) == 0
                with open(args.csv, "a") as f:
                    f.write(W.summary_csv(record, args.baseline_us, header=new))
        return correctness

    verdicts = [run_case(cfg) for cfg in cases]
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0 if "failed" not in verdicts else 1


def sweep(buf, cfg, x, handle, back, routes, rank, world, args, fresh):
    """Cached dispatch and combine under explicit SM splits (engine level: the public API only splits the combine)."""
    import torch.distributed as dist

    eng, plan = buf.engine, handle._plan
    mode = 2 if cfg.dtype == "fp8" else 0
    local = cfg.experts // world
    dst = torch.where(routes[rank][0] >= 0, torch.div(routes[rank][0], local, rounding_mode="floor"), torch.full_like(routes[rank][0], -1))
    remote_rows = sum(int((dst == d).any(dim=1).sum()) for d in range(world) if d != rank)
    out_bytes = {"dispatch": remote_rows * (cfg.hidden * 2 if mode == 0 else cfg.hidden + cfg.hidden // 128 * 4),
                 "combine": remote_rows * cfg.hidden * 2}

    def timed(fn, iters=10):
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
        t = torch.tensor([s.elapsed_time(e) / iters * 1e3], device=x.device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def say(**kw):
        if rank == 0:
            print(json.dumps(kw), flush=True)

    limit = max(2, eng.sm_count)
    for blocks in args.sweep_blocks:
        blocks = min(blocks, limit)
        for frac in args.sweep_fractions:
            send = min(blocks - 1, max(1, round(blocks * frac)))
            for op, fn in (("dispatch", lambda: eng.dispatch([x], [plan], mode, split=(send, blocks - send))),
                           ("combine", lambda: eng.combine([back], [plan], [None], split=(send, blocks - send)))):
                us = timed(fn)
                say(sweep=op, blocks=blocks, nvlink_side_blocks=send, us=round(us, 1),
                    nvlink_out_GBps=round(out_bytes[op] / (us * 1e-6) / 1e9, 1))
    if args.device_profile:
        eng.enable_device_profile(True)
        fresh()                                   # the routing layout pass stamps its phases
        say(profile="notify", phases_us={k: round(v, 1) for k, v in eng.phase_stamps("notify").items()})
        eng.dispatch([x], [plan], mode)
        eng.combine([back], [plan], [None])
        notify_stamps = eng.phase_stamps("notify")
        prof = eng.pop_device_profile()
        eng.enable_device_profile(False)
        if args.trace:
            from deepep_b200.utils import trace as TR

            # one timeline per rank: notify, then dispatch, then combine, laid end to end (they ran one after the other)
            mine, at = TR.from_phase_stamps("notify", notify_stamps, rank), max(list(notify_stamps.values()) + [0.0])
            for op in ("dispatch", "combine"):
                part = {k: v for k, v in prof.items() if k[0] == op}
                mine += [dict(e, pid=rank) for e in TR.from_device_profile(part, offset_us=at)]
                at += max([b["end_us"] for blocks in part.values() for b in blocks] + [0.0])
            everyone = buf.control.all_gather_object(mine)
            if rank == 0:
                TR.write_trace(args.trace, [e for part in everyone for e in part])
                say(trace=args.trace, spans=sum(len(part) for part in everyone))
        for (op, _), blocks in prof.items():
            for side in sorted({b["role"] for b in blocks}):
                sel = [b for b in blocks if b["role"] == side]
                say(profile=op, side=side, blocks=len(sel), first_start_us=round(min(b["start_us"] for b in sel), 1),
                    last_end_us=round(max(b["end_us"] for b in sel), 1),
                    mean_busy_us=round(sum(b["end_us"] - b["start_us"] for b in sel) / len(sel), 1),
                    **{k: round(sum(b[k] for b in sel) / len(sel), 1) for k in ("meta_us", "wait_us", "data_us", "publish_us")},
                    rows=sum(b["rows"] for b in sel))


if __name__ == "__main__":
    sys.exit(main())
