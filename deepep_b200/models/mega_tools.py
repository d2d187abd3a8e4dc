"""Fused-MoE tooling: input preflight, accuracy metrics and gate, cached CPU goldens.

Parity: ``experiments/megamoe/python/deep_ep_experimental/megamoe/validation.py`` (``check_routing``,
``collective_check``), ``golden.py`` (``contract`` / ``cache_path`` / ``digest`` / ``load`` / ``save`` / ``generate`` /
``compare``) and the accuracy half of ``benchmark.py`` of the reference.  The golden itself is computed by
:func:`deepep_b200.oracle.megamoe.mega_moe_reference` on the CPU and cached on disk keyed by everything that
determines it, so that repeated accuracy runs at large shapes do not recompute it.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..oracle import megamoe as O


# ------------------------------------------------------------------------------------------------ preflight
def check_routing(indices: Sequence[Sequence[int]], weights: Sequence[Sequence[float]], num_experts: int, num_topk: int,
                  allow_masked: bool = True) -> None:
    """Validates host lists taken from the actual input tensors (an explicit preflight, never a scan in the kernel).

    ``allow_masked``: ``-1`` marks an unused slot (the kernels skip it); the reference rejects it.
    """
    if len(indices) != len(weights):
        raise ValueError("routing ids and weights have different batch sizes")
    for token, (ids, probs) in enumerate(zip(indices, weights)):
        if len(ids) != num_topk or len(probs) != num_topk:
            raise ValueError(f"token={token}: routing width must equal top-k={num_topk}")
        for e in ids:
            if type(e) is not int or not (0 <= e < num_experts or (allow_masked and e == -1)):
                raise ValueError(f"token={token}: expert ids must be in [0,{num_experts})" + (" or -1" if allow_masked else ""))
        real = [e for e in ids if e >= 0]
        if len(set(real)) != len(real):
            raise ValueError(f"token={token}: duplicate expert ids are unsupported")
        if any(not math.isfinite(v) for v in probs):
            raise ValueError(f"token={token}: route weights must be finite")


def collective_check(control, stage: str, error: Optional[str], signature=None) -> None:
    """All ranks exchange (error, signature): raises everywhere if any rank failed or the signatures differ.

    ``control`` is anything with ``all_gather_object`` (:class:`deepep_b200.parallel.runtime.ControlPlane`) or
    ``all_gather(obj, tag)`` (:class:`deepep_b200.parallel.store.StoreGroup`).
    """
    if hasattr(control, "all_gather_object"):
        peers = control.all_gather_object((error, signature))
    else:
        peers = control.all_gather((error, signature), f"check:{stage}")
    failures = [f"rank={r}: {v[0]}" for r, v in enumerate(peers) if v[0]]
    if failures:
        raise ValueError(f"MegaMoE {stage} failed: " + "; ".join(failures))
    if any(v[1] != peers[0][1] for v in peers):
        raise ValueError(f"MegaMoE {stage}: ranks disagree: " + "; ".join(f"rank={r}: {v[1]}" for r, v in enumerate(peers)))


# ------------------------------------------------------------------------------------------------ metrics
def error_metrics(actual: torch.Tensor, expected: torch.Tensor) -> Dict[str, float]:
    """MARE (max relative error), MERE (mean relative error), RMSE and max absolute error, in fp32.

    Relative errors use ``max(|expected|, 1)`` as denominator, the convention of the reference's mixed-error gate.
    """
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    if a.shape != e.shape:
        raise ValueError(f"shape mismatch: {tuple(a.shape)} against {tuple(e.shape)}")
    if a.numel() == 0:
        return dict(mare=0.0, mere=0.0, rmse=0.0, max_abs=0.0, nonfinite=0.0)
    bad = ~torch.isfinite(a)
    diff = (a - e).abs()
    diff[bad] = float("inf")
    rel = diff / e.abs().clamp(min=1.0)
    finite = rel[~bad]
    return dict(mare=float(rel.max()), mere=float(finite.mean()) if finite.numel() else float("inf"),
                rmse=float(((a - e)[~bad] ** 2).mean().sqrt()) if finite.numel() else float("inf"),
                max_abs=float(diff.max()), nonfinite=float(bad.float().mean()))


def compare(actual: torch.Tensor, expected: torch.Tensor, *, diff_thd: float = 0.01, pct_thd: float = 0.05,
            max_diff: float = 0.1) -> Dict[str, float]:
    """The mixed-error gate: at most ``pct_thd`` of the elements may be off by more than ``diff_thd`` (relative, with
    ``max(|expected|, 1)``), none by more than ``max_diff``.  Returns the metrics plus ``ok`` and ``bad_fraction``."""
    m = error_metrics(actual, expected)
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    rel = (a - e).abs() / e.abs().clamp(min=1.0)
    rel[~torch.isfinite(a)] = float("inf")
    m["bad_fraction"] = float((rel > diff_thd).float().mean()) if rel.numel() else 0.0
    m["ok"] = bool(m["bad_fraction"] <= pct_thd and m["mare"] <= max_diff)
    return m


# ------------------------------------------------------------------------------------------------ device timer
TIMER_SLOTS = ("start", "handshake", "layout", "pull", "gemm", "finish_sync", "end")


def parse_timer(timer: torch.Tensor) -> Dict[str, float]:
    """Per-phase breakdown of one fused-kernel launch from the records of ``SymmBuffer.allocate_timer()``.

    Every CTA stamps ``%globaltimer`` at: kernel start, inputs quantised + handshake done, routing layout done, its pull
    warps done, its GEMM tile loop done, finish handshake done, end.  The result holds, in microseconds, the time
    from the earliest start to the latest stamp of each boundary (so the phases add up to ``total_us``), plus the
    spread of the CTAs' GEMM end (``gemm_tail_us``: how long the slowest CTA worked after the fastest was done) and
    ``mma_thread_wait_share``: the share of its tile loop that the thread issuing the MMAs spent waiting for operands.
    Parity: the reference's timer tooling (``timer/protocol.py``, ``timer/parse_timer_csv.py``, ``timer/breakdown.py``).
    """
    rec = timer.detach().cpu().to(torch.int64)
    rec = rec[rec[:, 0] > 0]
    if rec.numel() == 0:
        return dict(ctas=0, total_us=0.0)
    t0 = int(rec[:, 0].min())
    last = {name: (int(rec[:, i][rec[:, i] > 0].max()) - t0) / 1e3 if bool((rec[:, i] > 0).any()) else 0.0
            for i, name in enumerate(TIMER_SLOTS)}
    gemm_ends = rec[:, 4][rec[:, 4] > 0]
    out = dict(ctas=int(rec.shape[0]), total_us=last["end"],
               handshake_us=last["handshake"], layout_us=max(0.0, last["layout"] - last["handshake"]),
               pull_done_us=last["pull"], gemm_us=max(0.0, last["gemm"] - last["layout"]),
               finish_sync_us=max(0.0, last["finish_sync"] - last["gemm"]), reduce_us=max(0.0, last["end"] - last["finish_sync"]),
               gemm_tail_us=(int(gemm_ends.max()) - int(gemm_ends.min())) / 1e3 if gemm_ends.numel() else 0.0)
    if rec.shape[1] > 7:      # word 7: cycles / 16 of the thread that issues the MMAs, (waiting for operands) << 32 | (its whole tile loop)
        word = rec[:, 7]
        word = word[word != 0]
        if word.numel():
            waited, total = (word >> 32) & 0xffffffff, word & 0xffffffff
            out["mma_thread_wait_share"] = float(waited.sum()) / max(float(total.sum()), 1.0)
    return out


# ------------------------------------------------------------------------------------------------ model configurations
MODEL_FIELDS = ("hidden", "intermediate_hidden", "num_experts", "num_topk", "num_shared_experts")


def load_model_config(path: str) -> Dict:
    """A benchmark configuration in the reference's schema (``configs/*.json`` of its megamoe package):
    ``{"schema_version": 1, "model": {hidden, intermediate_hidden, num_experts, num_topk, num_shared_experts},
    "bs_values": [...], "warmup": n, "iters": n, "seed": n}``.  Unknown keys, missing keys and values this library cannot
    run (hidden not a multiple of 256, intermediate size not a multiple of 128, top-k plus shared experts above 16)
    are errors; returns the validated dictionary."""
    with open(path) as fh:
        cfg = json.load(fh)
    if not isinstance(cfg, dict) or cfg.get("schema_version") != 1:
        raise ValueError("a model configuration is a JSON object with schema_version 1")
    unknown = set(cfg) - {"schema_version", "model", "bs_values", "warmup", "iters", "seed"}
    if unknown:
        raise ValueError("unknown configuration fields: " + ", ".join(sorted(unknown)))
    model = cfg.get("model")
    if not isinstance(model, dict) or set(model) != set(MODEL_FIELDS):
        raise ValueError("model must hold exactly " + ", ".join(MODEL_FIELDS))
    if any(type(model[k]) is not int or model[k] < 0 for k in MODEL_FIELDS):
        raise ValueError("model fields are nonnegative integers")
    if model["hidden"] <= 0 or model["hidden"] % 256 or model["intermediate_hidden"] <= 0 or model["intermediate_hidden"] % 128:
        raise ValueError("hidden must be a positive multiple of 256 and intermediate_hidden of 128")
    if not 1 <= model["num_topk"] <= model["num_experts"] or model["num_topk"] + model["num_shared_experts"] > 16:
        raise ValueError("num_topk must be in [1, num_experts] and num_topk + num_shared_experts at most 16")
    sizes = cfg.get("bs_values")
    if not isinstance(sizes, list) or not sizes or any(type(b) is not int or not 1 <= b <= 16384 for b in sizes):
        raise ValueError("bs_values is a non-empty list of batch sizes in [1, 16384]")
    out = dict(schema_version=1, model={k: model[k] for k in MODEL_FIELDS}, bs_values=list(sizes))
    for key, default, low in (("warmup", 3, 0), ("iters", 10, 1), ("seed", 0, 0)):
        value = cfg.get(key, default)
        if type(value) is not int or value < low:
            raise ValueError(f"{key} must be an integer >= {low}")
        out[key] = value
    return out


# ------------------------------------------------------------------------------------------------ goldens
def contract(*, world: int, tokens: Sequence[int], hidden: int, intermediate: int, experts: int, topk: int, seed: int,
             routing: str = "random") -> Dict:
    """Everything that determines a golden; its digest names the cache files."""
    return dict(version=1, world=int(world), tokens=[int(t) for t in tokens], hidden=int(hidden), intermediate=int(intermediate),
                experts=int(experts), topk=int(topk), seed=int(seed), routing=str(routing))


def digest(spec: Dict) -> str:
    return hashlib.sha256(json.dumps(spec, sort_keys=True).encode()).hexdigest()[:16]


def cache_path(directory: str, spec: Dict, rank: int) -> str:
    return os.path.join(directory, f"megamoe_golden_{digest(spec)}_rank{rank}.pt")


def make_case(spec: Dict):
    """Deterministic inputs of a contract: per-rank (codes, scales), topk_idx, topk_weights and the two weight sets."""
    E, H, I, K = spec["experts"], spec["hidden"], spec["intermediate"], spec["topk"]
    l1, l2 = O.make_weights(E, H, I, spec["seed"])
    xs, idx, ws = [], [], []
    for r, t in enumerate(spec["tokens"]):
        g = torch.Generator().manual_seed(spec["seed"] * 1000 + r)
        xs.append(O.quantize_mxfp8(torch.randn((t, H), generator=g)))
        if spec["routing"] == "balanced":
            base = (torch.arange(t * K) + r) % E
            idx.append(base.view(t, K).to(torch.int64))
        else:
            idx.append(torch.rand((t, E), generator=g).topk(K, dim=1).indices)
        ws.append(torch.softmax(torch.randn((t, K), generator=g), dim=1))
    return xs, idx, ws, l1, l2


def generate(spec: Dict, directory: Optional[str] = None) -> List[torch.Tensor]:
    """Computes (or loads) the golden outputs of every rank; writes them to ``directory`` when given."""
    if directory:
        paths = [cache_path(directory, spec, r) for r in range(spec["world"])]
        if all(os.path.exists(p) for p in paths):
            loaded = [torch.load(p) for p in paths]
            if all(item["spec"] == spec for item in loaded):
                return [item["output"] for item in loaded]
    xs, idx, ws, l1, l2 = make_case(spec)
    outs = O.mega_moe_reference(xs, idx, ws, l1, l2, spec["experts"])
    if directory:
        os.makedirs(directory, exist_ok=True)
        for r, out in enumerate(outs):
            tmp = cache_path(directory, spec, r) + f".tmp{os.getpid()}"
            torch.save(dict(spec=spec, output=out), tmp)
            os.replace(tmp, cache_path(directory, spec, r))
    return outs


def accuracy_report(actual: Sequence[torch.Tensor], spec: Dict, directory: Optional[str] = None) -> Tuple[bool, List[Dict]]:
    """Compares every rank's output with the golden of ``spec``; returns (all ok, per-rank metrics)."""
    golden = generate(spec, directory)
    rows = [compare(a, g) for a, g in zip(actual, golden)]
    return all(r["ok"] for r in rows), rows


__all__ = ["accuracy_report", "cache_path", "check_routing", "collective_check", "compare", "contract", "digest",
           "error_metrics", "generate", "load_model_config", "make_case", "parse_timer"]
