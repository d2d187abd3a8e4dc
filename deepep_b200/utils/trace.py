"""Timelines of the device-side records as Chrome-trace / Perfetto JSON.

The profile instantiations of the kernels leave three kinds of records: per-block phase records of the
high-throughput dispatch / combine (``CudaEngine.pop_device_profile``), phase stamps of block 0 of notify and of the
low-latency kernels (``CudaEngine.phase_stamps``), and the per-CTA ``%globaltimer`` stamps of the fused MoE kernel
(``SymmBuffer.allocate_timer``).  The functions here turn each into trace events (one process per rank, one thread
per block / CTA) that ``chrome://tracing`` and ``ui.perfetto.dev`` display, and ``write_trace`` stores them.

Parity: the reference's trace tooling (``experiments/megamoe/python/deep_ep_experimental/megamoe/timer/trace_parser.py``
and the Perfetto export of ``tests/elastic/notify_profile.py``).
"""
from __future__ import annotations

import json
from typing import Dict, Iterable, List, Mapping, Optional, Sequence

Event = Dict[str, object]


def span(name: str, start_us: float, end_us: float, rank: int = 0, track: int = 0, category: str = "deepep",
         args: Optional[Mapping[str, object]] = None) -> Event:
    """One complete event ("ph": "X"); times in microseconds, a span that ends before it starts has length zero."""
    ev: Event = {"name": name, "cat": category, "ph": "X", "ts": float(start_us), "dur": max(0.0, float(end_us) - float(start_us)),
                 "pid": int(rank), "tid": int(track)}
    if args:
        ev["args"] = dict(args)
    return ev


def from_device_profile(profile: Mapping, offset_us: float = 0.0) -> List[Event]:
    """``profile`` is what ``CudaEngine.pop_device_profile()`` returns: ``{(op, rank index): [per-block dict]}``.
    Every block becomes one span named after its role, carrying its phase totals as arguments."""
    events: List[Event] = []
    for (op, rank), blocks in sorted(profile.items()):
        for track, b in enumerate(blocks):
            extra = {k: round(float(b[k]), 3) for k in ("meta_us", "wait_us", "data_us", "publish_us") if k in b}
            extra["rows"] = int(b.get("rows", 0))
            events.append(span(f"{op}:{b['role']}", offset_us + b["start_us"], offset_us + b["end_us"], rank, track, op, extra))
    return events


def from_phase_stamps(op: str, stamps: Mapping[str, float], rank: int = 0, track: int = 0, offset_us: float = 0.0) -> List[Event]:
    """``stamps``: phase name -> microseconds since kernel start at which the phase was complete (``phase_stamps``).
    Phases are laid end to end in the order of their stamps; phases that were never stamped (zero) are left out."""
    events: List[Event] = []
    at = 0.0
    for name, t in sorted(((n, float(v)) for n, v in stamps.items() if float(v) > 0), key=lambda item: item[1]):
        events.append(span(f"{op}:{name}", offset_us + at, offset_us + t, rank, track, op))
        at = max(at, t)
    return events


MEGA_PHASES = (("handshake", 0, 1), ("layout", 1, 2), ("pull", 2, 3), ("gemm", 2, 4), ("finish_sync", 4, 5), ("reduce", 5, 6))


def from_mega_timer(timer, rank: int = 0) -> List[Event]:
    """``timer``: the int64 ``[CTAs, words]`` tensor (or nested list) a fused-MoE launch filled.  Every CTA becomes a
    thread with its phases as spans (nanosecond stamps relative to the earliest start); the pull warps work beside
    the GEMM warps, so their span goes to a second thread of the same CTA."""
    rows = timer.detach().cpu().tolist() if hasattr(timer, "detach") else [list(r) for r in timer]
    rows = [(i, r) for i, r in enumerate(rows) if r[0] > 0]
    if not rows:
        return []
    t0 = min(r[0] for _, r in rows)
    events: List[Event] = []
    for cta, r in rows:
        for name, a, b in MEGA_PHASES:
            if r[a] > 0 and r[b] > 0:
                track = 2 * cta + (1 if name == "pull" else 0)
                args = None
                if name == "gemm" and len(r) > 7 and r[7]:
                    waited, total = (r[7] >> 32) & 0xffffffff, r[7] & 0xffffffff
                    args = {"mma_thread_wait_share": round(waited / max(total, 1), 4)}
                events.append(span(f"mega_moe:{name}", (r[a] - t0) / 1e3, (r[b] - t0) / 1e3, rank, track, "mega_moe", args))
    return events


def chrome_trace(events: Iterable[Event], rank_names: Optional[Mapping[int, str]] = None) -> Dict[str, object]:
    """The JSON object of the trace-event format: the spans sorted by time plus one name record per process."""
    spans = sorted(events, key=lambda e: (e["pid"], e["tid"], e["ts"]))
    meta = [{"name": "process_name", "ph": "M", "pid": pid, "tid": 0,
             "args": {"name": (rank_names or {}).get(pid, f"rank {pid}")}} for pid in sorted({int(e["pid"]) for e in spans})]
    return {"displayTimeUnit": "ns", "traceEvents": meta + spans}


def write_trace(path: str, events: Iterable[Event], rank_names: Optional[Mapping[int, str]] = None) -> str:
    with open(path, "w") as fh:
        json.dump(chrome_trace(events, rank_names), fh)
    return path


def summarize(events: Sequence[Event]) -> Dict[str, Dict[str, float]]:
    """Per span name: count, total, mean and maximum duration in microseconds (the table printed next to a trace)."""
    out: Dict[str, Dict[str, float]] = {}
    for e in events:
        row = out.setdefault(str(e["name"]), {"count": 0, "total_us": 0.0, "max_us": 0.0})
        row["count"] += 1
        row["total_us"] += float(e["dur"])
        row["max_us"] = max(row["max_us"], float(e["dur"]))
    for row in out.values():
        row["mean_us"] = row["total_us"] / row["count"]
    return out


__all__ = ["chrome_trace", "from_device_profile", "from_mega_timer", "from_phase_stamps", "span", "summarize", "write_trace"]
