"""Benchmark workloads as validated JSON configurations, logical byte accounting and versioned result records.

Parity: ``benchmarks/_config.py:14-126`` (strict configuration dataclass, fingerprint, logical traffic) and
``benchmarks/_utils.py:18-149`` (schema-versioned records, rank-max aggregation with nearest-rank percentiles,
result directories that are never overwritten) of the reference.  ``benchmarks/bench_ep.py`` runs a configuration.
"""
from __future__ import annotations

import csv
import hashlib
import io
import itertools
import json
import math
import os
import time
from dataclasses import asdict, dataclass, fields
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .testing import aggregate_rank_max, bandwidth_gbps

SCHEMA_VERSION = 1
MAX_CONFIG_BYTES = 65536
MAX_MATRIX_CASES = 4096
TIMING = {
    "clock": "cuda_events_on_the_launching_stream",
    "rank_aggregation": "max_per_iteration_then_statistics",
    "percentile": "nearest_rank",
    "includes": ["notify_for_fresh_dispatch", "kernel_time", "stream_ordering_events"],
    "excludes": ["input_generation", "correctness", "host_copies"],
    "cache_policy": "l2_flush_between_iterations",
}
_CHOICES = {
    "operation": ("dispatch", "combine", "roundtrip"),
    "dtype": ("bf16", "fp8"),                       # dispatch payload; fp8 = e4m3 with fp32 scales per 128, quantised in the kernel
    "layout": ("expanded", "rank"),                 # rows per (token, slot) sorted by expert, or one row per received token
    "dispatch_mode": ("fresh", "cached"),           # with or without the routing-layout pass
    "route": ("balanced", "skew", "masked", "grouped", "next_rank"),
}
_LIMITS = {"world_size": (1, 8), "hidden": (128, 7168), "topk": (1, 16), "experts": (1, 1024), "seed": (0, 2 ** 31 - 1),
           "warmup": (0, 10000), "iterations": (1, 10000), "alignment": (1, 128)}


@dataclass(frozen=True)
class WorkloadConfig:
    operation: str = "roundtrip"
    dtype: str = "bf16"
    layout: str = "expanded"
    dispatch_mode: str = "cached"
    world_size: int = 1
    tokens_per_rank: Tuple[int, ...] = (64,)
    hidden: int = 256
    topk: int = 2
    experts: int = 8
    alignment: int = 1
    with_weights: bool = True
    route: str = "balanced"
    seed: int = 0
    warmup: int = 3
    iterations: int = 10

    def validate(self) -> "WorkloadConfig":
        for name, allowed in _CHOICES.items():
            if getattr(self, name) not in allowed:
                raise ValueError(f"{name} must be one of {allowed}")
        for name, (lo, hi) in _LIMITS.items():
            v = getattr(self, name)
            if type(v) is not int or not lo <= v <= hi:
                raise ValueError(f"{name} must be an integer in [{lo}, {hi}]")
        if type(self.with_weights) is not bool:
            raise ValueError("with_weights must be boolean")
        t = self.tokens_per_rank
        if not isinstance(t, (list, tuple)) or len(t) != self.world_size or any(type(v) is not int or not 0 <= v <= 16384 for v in t):
            raise ValueError("tokens_per_rank must hold one integer in [0, 16384] per rank")
        if sum(t) < 1:
            raise ValueError("at least one token is needed")
        if self.experts % self.world_size or self.topk > self.experts:
            raise ValueError("experts must divide across ranks and topk must not exceed experts")
        if self.hidden % 128:
            raise ValueError("hidden must be a multiple of 128")
        if self.alignment > 1 and self.layout != "expanded":
            raise ValueError("expert alignment applies to the expanded layout")
        if self.operation == "combine" and self.dispatch_mode == "fresh":
            raise ValueError("dispatch_mode=fresh applies to dispatch or roundtrip")
        if self.world_size * self.iterations > 1_000_000:
            raise ValueError("at most 1000000 rank samples are kept")
        return self

    def to_dict(self) -> Dict:
        d = asdict(self)
        d["tokens_per_rank"] = list(self.tokens_per_rank)
        return d

    @classmethod
    def from_dict(cls, data) -> "WorkloadConfig":
        if not isinstance(data, dict):
            raise ValueError("a configuration is a JSON object")
        unknown = set(data) - {f.name for f in fields(cls)}
        if unknown:
            raise ValueError("unknown configuration fields: " + ", ".join(sorted(unknown)))
        data = dict(data)
        if isinstance(data.get("tokens_per_rank"), list):
            data["tokens_per_rank"] = tuple(data["tokens_per_rank"])
        return cls(**data).validate()

    @classmethod
    def from_json(cls, path: str) -> "WorkloadConfig":
        if os.path.getsize(path) > MAX_CONFIG_BYTES:
            raise ValueError(f"configuration file is larger than {MAX_CONFIG_BYTES} bytes")
        with open(path) as f:
            return cls.from_dict(json.load(f, object_pairs_hook=_no_duplicate_keys))

    def fingerprint(self) -> str:
        return hashlib.sha256(json.dumps(self.to_dict(), sort_keys=True).encode()).hexdigest()


def _no_duplicate_keys(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise ValueError(f"duplicate configuration key {k!r}")
        out[k] = v
    return out


# ------------------------------------------------------------------------------------------------ routes and traffic
def make_routes(cfg: WorkloadConfig, rank: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Deterministic ``(topk_idx int64 [T, K], topk_weights fp32 [T, K])`` of one rank (CPU tensors)."""
    T, K, E = cfg.tokens_per_rank[rank], cfg.topk, cfg.experts
    g = torch.Generator().manual_seed(cfg.seed * 1009 + rank)
    if cfg.route == "balanced":
        start = (torch.arange(T) * K + rank) % E
        idx = (start.unsqueeze(1) + torch.arange(K).unsqueeze(0) * max(1, E // K)) % E if K * max(1, E // K) <= E else \
            torch.rand((T, E), generator=g).topk(K, dim=1).indices
    elif cfg.route == "skew":         # half of the probability mass on the first eighth of the experts
        p = torch.ones(E)
        p[:max(1, E // 8)] = 8.0
        idx = torch.multinomial(p.expand(max(T, 1), E), K, generator=g)[:T]
    elif cfg.route == "grouped":      # group-limited routing: top-4 of 8 expert groups, then top-k inside them
        groups = 8 if E % 8 == 0 and E >= 8 * K else 1
        scores = torch.rand((T, E), generator=g)
        if groups > 1:
            best = scores.view(T, groups, E // groups).amax(2).topk(min(4, groups), dim=1).indices
            mask = torch.zeros((T, groups), dtype=torch.bool).scatter_(1, best, True).repeat_interleave(E // groups, dim=1)
            scores = scores.masked_fill(~mask, -1.0)
        idx = scores.topk(K, dim=1).indices
    elif cfg.route == "next_rank":    # link stress: every token goes only to experts of the next rank
        local = E // cfg.world_size
        base = ((rank + 1) % cfg.world_size) * local
        idx = base + torch.rand((T, local), generator=g).topk(min(K, local), dim=1).indices
        if idx.shape[1] < K:
            idx = torch.cat([idx, torch.full((T, K - idx.shape[1]), -1, dtype=idx.dtype)], dim=1)
    else:                             # masked: random routes with a quarter of the slots disabled
        idx = torch.rand((T, E), generator=g).topk(K, dim=1).indices
        idx[torch.rand((T, K), generator=g) < 0.25] = -1
    idx = idx.to(torch.int64).reshape(T, K)
    return idx, torch.softmax(torch.randn((T, K), generator=g), dim=1)


def traffic(cfg: WorkloadConfig, routes: Sequence[torch.Tensor]) -> Dict[str, float]:
    """Logical bytes of one iteration over all ranks: every (token, destination rank) row once per direction."""
    local = cfg.experts // cfg.world_size
    rows = 0
    for idx in routes:
        dst = torch.where(idx >= 0, torch.div(idx, local, rounding_mode="floor"), torch.full_like(idx, -1))
        rows += sum(int((dst == d).any(dim=1).sum()) for d in range(cfg.world_size))
    row_out = cfg.hidden * 2 if cfg.dtype == "bf16" else cfg.hidden + cfg.hidden // 128 * 4
    row_back = cfg.hidden * 2
    per_op = {"dispatch": rows * row_out, "combine": rows * row_back}
    per_op["roundtrip"] = per_op["dispatch"] + per_op["combine"]
    return {"rank_rows": rows, "effective_bytes": float(per_op[cfg.operation])}


# ------------------------------------------------------------------------------------------------ records
def plan(cfg: WorkloadConfig) -> Dict:
    cfg.validate()
    return {"schema_version": SCHEMA_VERSION, "status": "planned", "config": cfg.to_dict(), "config_fingerprint": cfg.fingerprint(),
            "timing": dict(TIMING), "correctness_result": "not_run"}


def complete(record: Dict, rank_samples_us: Sequence[Sequence[float]], effective_bytes: float, correctness: str) -> Dict:
    """Fills a planned record with the gathered per-rank samples (microseconds) and their statistics."""
    cfg = WorkloadConfig.from_dict(record["config"])
    if len(rank_samples_us) != cfg.world_size or any(len(r) != cfg.iterations for r in rank_samples_us):
        raise ValueError("incomplete rank samples")
    stats = aggregate_rank_max(rank_samples_us)
    out = dict(record)
    out.update(status="measured", rank_samples_us=[list(map(float, r)) for r in rank_samples_us], statistics=stats,
               effective_bytes=effective_bytes, bandwidth_gbps=bandwidth_gbps(effective_bytes, stats["mean_rank_max_us"]),
               bandwidth_statistic="effective_bytes_over_mean_rank_max_latency", correctness_result=correctness,
               measured_at=time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()))
    return out


def write_result(directory: str, record: Dict) -> str:
    """Writes ``<directory>/<fingerprint prefix>_<n>.json``; an existing file is never overwritten."""
    os.makedirs(directory, exist_ok=True)
    stem = record["config_fingerprint"][:12]
    for n in range(10000):
        path = os.path.join(directory, f"{stem}_{n:04d}.json")
        try:
            fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_EXCL)
        except FileExistsError:
            continue
        with os.fdopen(fd, "w") as f:
            json.dump(record, f, indent=1, sort_keys=True)
        return path
    raise RuntimeError("too many results for one configuration in this directory")


def verify_record(record: Dict) -> Dict:
    """Checks a measured record against itself: the configuration must validate and hash to the stored fingerprint, and
    the statistics and the bandwidth must follow from the stored per-rank samples (they are recomputed, never trusted).
    Returns the recomputed statistics."""
    cfg = WorkloadConfig.from_dict(record.get("config"))
    if record.get("config_fingerprint") != cfg.fingerprint():
        raise ValueError("the record's fingerprint does not belong to its configuration")
    if record.get("status") != "measured":
        raise ValueError("only measured records carry statistics")
    samples = record.get("rank_samples_us")
    if not isinstance(samples, list) or len(samples) != cfg.world_size or any(len(r) != cfg.iterations for r in samples):
        raise ValueError("incomplete rank samples")
    stats = aggregate_rank_max(samples)
    for name, value in stats.items():
        if abs(float(record["statistics"].get(name, float("nan"))) - value) > 1e-9 * max(1.0, abs(value)):
            raise ValueError(f"stored statistic {name} does not follow from the samples")
    want = bandwidth_gbps(float(record["effective_bytes"]), stats["mean_rank_max_us"])
    if abs(float(record["bandwidth_gbps"]) - want) > 1e-9 * max(1.0, want):
        raise ValueError("stored bandwidth does not follow from the samples")
    return stats


CSV_FIELDS = ("config_fingerprint", "operation", "dtype", "layout", "dispatch_mode", "world_size", "tokens_per_rank", "hidden",
              "topk", "experts", "route", "iterations", "latency_mean_us", "latency_p50_us", "latency_p95_us", "latency_max_us",
              "effective_bytes", "bandwidth_gbps", "correctness_result", "baseline_latency_us", "speedup")


def summary_csv(record: Dict, baseline_latency_us: Optional[float] = None, header: bool = True) -> str:
    """One CSV row (after the header line) for a measured record; ``baseline_latency_us`` (a number measured elsewhere for
    the same configuration) fills the last two columns, which stay empty without it."""
    stats, cfg = verify_record(record), record["config"]
    row = {name: cfg[name] for name in CSV_FIELDS if name in cfg}
    row.update(config_fingerprint=record["config_fingerprint"], tokens_per_rank=" ".join(map(str, cfg["tokens_per_rank"])),
               latency_mean_us=stats["mean_rank_max_us"], latency_p50_us=stats["p50_us"], latency_p95_us=stats["p95_us"],
               latency_max_us=stats["max_us"], effective_bytes=record["effective_bytes"], bandwidth_gbps=record["bandwidth_gbps"],
               correctness_result=record["correctness_result"], baseline_latency_us="", speedup="")
    if baseline_latency_us is not None:
        if not baseline_latency_us > 0:
            raise ValueError("a baseline latency is a positive number of microseconds")
        row.update(baseline_latency_us=float(baseline_latency_us), speedup=float(baseline_latency_us) / stats["mean_rank_max_us"])
    out = io.StringIO()
    writer = csv.DictWriter(out, fieldnames=CSV_FIELDS, lineterminator="\n")
    if header:
        writer.writeheader()
    writer.writerow(row)
    return out.getvalue()


def with_overrides(cfg: WorkloadConfig, assignments: Sequence[str]) -> WorkloadConfig:
    """``cfg`` with ``name=value`` assignments applied (values in JSON syntax; a bare word is a string), validated."""
    data = cfg.to_dict()
    for item in assignments:
        name, sep, text = item.partition("=")
        if not sep or name not in data:
            raise ValueError(f"override {item!r}: expected name=value with a configuration field's name")
        try:
            data[name] = json.loads(text, object_pairs_hook=_no_duplicate_keys)
        except json.JSONDecodeError:
            data[name] = text
    return WorkloadConfig.from_dict(data)


def expand_matrix(cfg: WorkloadConfig, axes: Sequence[str]) -> List[WorkloadConfig]:
    """Every combination of the values listed by ``name=[v1, v2, ...]`` axes applied to ``cfg`` (field names in sorted
    order, the last one varying fastest).  Each member is validated like a configuration file; combinations that give the
    same configuration are run once.  No axes: ``[cfg]``."""
    choices: Dict[str, list] = {}
    for item in axes:
        name, sep, text = item.partition("=")
        try:
            values = json.loads(text) if sep else None
        except json.JSONDecodeError:
            values = None
        if name not in cfg.to_dict() or not isinstance(values, list) or not values:
            raise ValueError(f"matrix axis {item!r}: expected name=[value, ...] with a configuration field's name")
        if name in choices:
            raise ValueError(f"matrix axis {name!r} is given twice")
        choices[name] = values
    names = sorted(choices)
    if math.prod(len(choices[n]) for n in names) > MAX_MATRIX_CASES:
        raise ValueError(f"a matrix holds at most {MAX_MATRIX_CASES} cases")
    out, seen = [], set()
    for combo in itertools.product(*(choices[n] for n in names)):
        try:
            member = WorkloadConfig.from_dict({**cfg.to_dict(), **dict(zip(names, combo))})
        except (ValueError, TypeError) as exc:
            raise ValueError(f"matrix member {dict(zip(names, combo))}: {exc}") from None
        if member.fingerprint() not in seen:
            seen.add(member.fingerprint())
            out.append(member)
    return out


__all__ = ["CSV_FIELDS", "SCHEMA_VERSION", "TIMING", "WorkloadConfig", "complete", "expand_matrix", "make_routes", "plan", "summary_csv", "traffic",
           "verify_record", "with_overrides", "write_result"]
