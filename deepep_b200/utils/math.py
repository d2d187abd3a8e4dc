"""Tensor and arithmetic helpers with the names DeepEP users expect.

Parity: ``deep_ep/utils/math.py`` of the reference (``calc_diff`` :17-23,
``per_token_cast_to_fp8`` :45-60, ``per_token_cast_back`` :64-79,
``inplace_unique`` :82-97, ``create_grouped_scores`` :100-106, hashes :109-131).
The fp8 recipe is the 1x128 block recipe: ``amax`` per 128 values clamped to
1e-4, ``scale = amax / 448``, ``q = e4m3(x * 448 / amax)``.
"""
from __future__ import annotations

from typing import Tuple

import torch

FP8_MAX = 448.0
FP8_BLOCK = 128


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - cosine-like similarity of ``x + 1`` and ``y + 1`` in float64."""
    a, b = x.double() + 1, y.double() + 1
    return float(1 - 2 * (a * b).sum() / (a * a + b * b).sum())


def safe_div(a, b):
    """``a / b`` with ``0 / 0 == 0`` (a rate over an empty interval); any other division by zero still raises."""
    if b:
        return a / b
    if a:
        raise ZeroDivisionError("division by zero")
    return 0


def ceil_div(x: int, y: int) -> int:
    """Smallest integer not below ``x / y``."""
    return -(-x // y)


def align(x: int, y: int) -> int:
    """``x`` rounded up to a multiple of ``y``."""
    return x + (-x) % y


def _pad_last(x: torch.Tensor, multiple: int) -> torch.Tensor:
    pad = align(x.shape[-1], multiple) - x.shape[-1]
    return torch.nn.functional.pad(x, (0, pad)) if pad else x


def per_token_cast_to_fp8(x: torch.Tensor, use_ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise ``[T, H]`` to e4m3 with one fp32 scale per 128 values.

    With ``use_ue8m0`` the scale is rounded up to a power of two, which is the
    form the block-scaled tensor-core path of MegaMoE consumes without loss.
    """
    assert x.dim() == 2, "x must be [tokens, hidden]"
    t, h = x.shape
    nblocks = align(h, FP8_BLOCK) // FP8_BLOCK
    blocks = _pad_last(x, FP8_BLOCK).view(t, nblocks, FP8_BLOCK)       # explicit sizes: an empty batch is legal
    amax = blocks.abs().float().amax(dim=2).clamp(1e-4)
    if use_ue8m0:
        scale = torch.exp2(torch.ceil(torch.log2(amax / FP8_MAX)))
        q = (blocks.float() / scale.unsqueeze(2)).to(torch.float8_e4m3fn)
    else:
        scale = amax / FP8_MAX
        q = (blocks * (FP8_MAX / amax.unsqueeze(2))).to(torch.float8_e4m3fn)
    return q.view(t, nblocks * FP8_BLOCK)[:, :h].contiguous(), scale


def per_token_cast_back(x_fp8: torch.Tensor, x_scales: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`per_token_cast_to_fp8` (bf16 result)."""
    if x_fp8.numel() == 0:
        return x_fp8.to(torch.bfloat16)
    assert x_fp8.dim() == 2
    t, h = x_fp8.shape
    if x_scales.dtype == torch.int:  # packed ue8m0 exponents
        x_scales = (x_scales.view(torch.uint8).to(torch.int) << 23).view(torch.float)
    vals = _pad_last(x_fp8, FP8_BLOCK).float().view(t, -1, FP8_BLOCK)
    out = vals * x_scales.reshape(t, -1, 1).float()
    return out.view(t, -1)[:, :h].to(torch.bfloat16).contiguous()


def inplace_unique(x: torch.Tensor, num_slots: int) -> None:
    """Replace every row by its distinct non-negative ids, descending, -1 padded."""
    assert x.dim() == 2
    present = torch.zeros((x.size(0), num_slots + 1), dtype=torch.bool, device=x.device)
    present.scatter_(1, x.masked_fill(x < 0, num_slots).long(), True)
    ids = torch.arange(num_slots, device=x.device, dtype=x.dtype).expand(x.size(0), -1)
    ids = torch.where(present[:, :num_slots], ids, torch.full_like(ids, -1))
    ids = torch.sort(ids, dim=-1, descending=True).values
    x.fill_(-1)
    n = min(num_slots, x.size(1))
    x[:, :n] = ids[:, :n]


def create_grouped_scores(scores: torch.Tensor, group_idx: torch.Tensor, num_groups: int) -> torch.Tensor:
    """Zero the scores of every expert whose group is not in ``group_idx``."""
    t, e = scores.shape
    keep = torch.zeros((t, num_groups), dtype=torch.bool, device=scores.device).scatter_(1, group_idx, True)
    return (scores.view(t, num_groups, -1) * keep.unsqueeze(-1)).view(t, e)


def _leaves(items):
    """Tensors of a nest of tuples and lists, depth first; anything else is skipped."""
    for item in items:
        if isinstance(item, torch.Tensor):
            yield item
        elif isinstance(item, (tuple, list)):
            yield from _leaves(item)


def hash_tensor(t: torch.Tensor) -> int:
    """Sum of the tensor's bytes read as int32 words (as bytes when their count is not a multiple of four): equal bits
    give equal values on every machine, so ranks can compare a number instead of a buffer."""
    flat = t.contiguous().reshape(-1).view(torch.uint8)
    words = flat.view(torch.int32) if flat.numel() % 4 == 0 else flat.to(torch.int32)
    return int(words.sum().item())


def hash_tensors(*tensors) -> int:
    """Exclusive-or of :func:`hash_tensor` over every tensor of the (nested) arguments."""
    value = 0
    for leaf in _leaves(tensors):
        value ^= hash_tensor(leaf)
    return value


def count_bytes(*tensors) -> int:
    """Bytes held by every tensor of the (nested) arguments; ``None`` entries count nothing."""
    return sum(leaf.numel() * leaf.element_size() for leaf in _leaves(tensors))


__all__ = [
    "align", "calc_diff", "ceil_div", "count_bytes", "create_grouped_scores", "hash_tensor",
    "hash_tensors", "inplace_unique", "per_token_cast_back", "per_token_cast_to_fp8", "safe_div",
]
