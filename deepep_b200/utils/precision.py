"""Accuracy metrics and the dual-reference acceptance rule for lossy paths (bf16 rounding, per-128 e4m3 dispatch).

The rule of the reference's test suite (``tests/utils/precision.py`` there): a result is judged against a float64 golden
*relative to a benchmark*, the same computation carried out in the data types of upstream DeepEP (bf16 activations, or
e4m3 values with one fp32 scale per 128 values restored to bf16).  With ``MARE`` the largest and ``MERE`` the mean
relative error and ``RMSE`` the root mean square error over the values that are not "small", the result passes level
``L2`` when its three errors are at most 2.0 / 1.2 / 1.2 times the benchmark's and its count of wrong small values at
most twice the benchmark's.  The exact kernels of this library (dispatch, combine) are checked for equality of bits
instead; this module serves lossy compositions (fp8 dispatch followed by a combine) and user code.

Everything here is tensor arithmetic in float64, so the numbers are those of the definition, not of a GPU data path.
"""
from __future__ import annotations

import math
from typing import Dict, Sequence

import torch

LEVEL_LIMITS = {"L0": (10.0, 2.0, 2.0), "L1": (5.0, 1.5, 1.5), "L2": (2.0, 1.2, 1.2)}      # MARE, MERE, RMSE ratios
DTYPE_POLICY = {
    "bfloat16": {"small_threshold": 2.0 ** -8, "small_error": 2.0 ** -16},
    "float8_e4m3fn": {"small_threshold": 2.0 ** -4, "small_error": 2.0 ** -6},
}


def to_bf16_values(x: torch.Tensor) -> torch.Tensor:
    """float64 -> the bf16 value nearest to its float32 rounding (two roundings, as a float32 program would do), as float64."""
    return x.double().float().bfloat16().double()


def _e4m3_table() -> torch.Tensor:
    values = []
    for bits in range(0x7F):                                    # 0x7F is NaN in e4m3fn; the largest finite value is 448
        exponent, mantissa = bits >> 3, bits & 7
        values.append(mantissa * 2.0 ** -9 if exponent == 0 else (1 + mantissa / 8.0) * 2.0 ** (exponent - 7))
    return torch.tensor(values, dtype=torch.float64)


_E4M3 = _e4m3_table()


def to_e4m3_values(x: torch.Tensor) -> torch.Tensor:
    """Nearest finite e4m3fn value of every element (ties to the even code, saturating at 448), as float64."""
    x = x.double()
    magnitude = x.abs().clamp(max=448.0)
    upper = torch.searchsorted(_E4M3, magnitude.contiguous()).clamp(max=_E4M3.numel() - 1)
    lower = (upper - 1).clamp(min=0)
    d_up, d_low = (_E4M3[upper] - magnitude).abs(), (magnitude - _E4M3[lower]).abs()
    take_upper = (d_up < d_low) | ((d_up == d_low) & (upper % 2 == 0))
    return torch.sign(x) * torch.where(take_upper, _E4M3[upper], _E4M3[lower])


def emulate_upstream(x: torch.Tensor, dtype: str) -> torch.Tensor:
    """What upstream DeepEP's dispatch delivers for float64 ``x`` ``[tokens, hidden]``, as float64: bf16 rounding, or
    (``float8_e4m3fn``) bf16 rounding, then per 128 values ``amax = max(|x|, 1e-4)``, code ``e4m3(x * (448 / amax))``,
    fp32 scale ``amax / 448``, and the product restored to bf16."""
    if dtype == "bfloat16":
        return to_bf16_values(x)
    if dtype != "float8_e4m3fn":
        raise ValueError(f"unsupported dtype: {dtype}")
    rows = to_bf16_values(x)
    tokens, hidden = rows.shape
    pad = (-hidden) % 128
    blocks = torch.nn.functional.pad(rows, (0, pad)).view(tokens, -1, 128)
    amax = blocks.abs().amax(dim=2, keepdim=True).clamp(min=1e-4)
    # tensor / tensor divisions: with a Python scalar on either side torch multiplies by a reciprocal, which is not the
    # correctly rounded quotient the definition asks for
    full = torch.full_like(amax, 448.0)
    scale = (amax / full).float().double()
    codes = to_e4m3_values(blocks * (full / amax))
    return to_bf16_values(codes * scale).view(tokens, -1)[:, :hidden]


def error_metrics(actual: torch.Tensor, golden: torch.Tensor, *, dtype: str) -> Dict[str, float]:
    """MARE / MERE / RMSE over the values whose golden magnitude reaches the data type's small-value threshold, and the
    number of smaller ones that are off by more than the small-value tolerance."""
    policy = DTYPE_POLICY[dtype]
    got, want = actual.double().reshape(-1), golden.double().reshape(-1)
    if got.shape != want.shape:
        raise ValueError("actual and golden shapes differ")
    if not bool(torch.isfinite(got).all() and torch.isfinite(want).all()):
        raise ValueError("precision comparison requires finite values")
    error = (got - want).abs()
    small = want.abs() < policy["small_threshold"]
    normal_error = error[~small]
    relative = normal_error / (want[~small].abs() + 1e-7)
    count = int(normal_error.numel())
    return dict(mare=float(relative.max()) if count else 0.0,
                mere=math.fsum(relative.tolist()) / count if count else 0.0,
                rmse=math.sqrt(math.fsum((normal_error * normal_error).tolist()) / count) if count else 0.0,
                small_error_count=int((error[small] > policy["small_error"]).sum()), normal_count=count,
                small_count=int(small.sum()))


def compare_dual(actual: torch.Tensor, benchmark: torch.Tensor, golden: torch.Tensor, *, dtype: str, level: str = "L2") -> Dict:
    """Judge ``actual`` against ``golden`` relative to ``benchmark`` (see the module text)."""
    if dtype not in DTYPE_POLICY or level not in LEVEL_LIMITS:
        raise ValueError("unknown dtype or precision level")
    got, ref = error_metrics(actual, golden, dtype=dtype), error_metrics(benchmark, golden, dtype=dtype)
    floor = DTYPE_POLICY[dtype]["small_error"]
    ratios = tuple(got[name] / max(ref[name], floor) for name in ("mare", "mere", "rmse"))
    small_ratio = got["small_error_count"] / max(ref["small_error_count"], 1)
    passed = all(r <= limit for r, limit in zip(ratios, LEVEL_LIMITS[level])) and small_ratio <= 2.0
    return dict(dtype=dtype, level=level, actual=got, benchmark=ref, ratios=dict(zip(("mare", "mere", "rmse"), ratios)),
                small_error_ratio=small_ratio, passed=bool(passed))


def bootstrap_median_recheck(ratios: Sequence[float], *, bootstrap_samples: int = 2000, seed: int = 0) -> Dict:
    """Second look at a borderline case from repeated runs: with at least 200 error ratios (actual / benchmark), the case
    passes when the 95 % bootstrap interval of their median reaches down to 1.0 or below; fewer samples never pass."""
    values = [float(v) for v in ratios]
    if not values or not all(math.isfinite(v) and v >= 0 for v in values):
        raise ValueError("recheck ratios must be nonempty, finite and nonnegative")
    if bootstrap_samples < 1:
        raise ValueError("bootstrap_samples must be positive")
    data = torch.tensor(values, dtype=torch.float64)
    median = float(data.quantile(0.5))
    if len(values) < 200:
        return dict(sample_count=len(values), median=median, ci_lower=float("nan"), ci_upper=float("nan"), passed=False,
                    reason="sample_count_below_200")
    g = torch.Generator().manual_seed(seed)
    picks = torch.randint(0, len(values), (bootstrap_samples, len(values)), generator=g)
    medians = data[picks].quantile(0.5, dim=1)
    lower, upper = float(medians.quantile(0.025)), float(medians.quantile(0.975))
    passed = lower <= 1.0
    return dict(sample_count=len(values), median=median, ci_lower=lower, ci_upper=upper, passed=passed,
                reason="ci_includes_or_below_1" if passed else "ci_lower_above_1")


__all__ = ["DTYPE_POLICY", "LEVEL_LIMITS", "bootstrap_median_recheck", "compare_dual", "emulate_upstream", "error_metrics",
           "to_bf16_values", "to_e4m3_values"]
