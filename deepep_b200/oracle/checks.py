"""Order-independent comparison of a dispatch / combine result with the oracle.

The kernels of this library place rows deterministically, so its own tests compare bits position by position.  A
checker for *any* implementation of the same contract (another build, a different schedule) must not: within one
expert's segment of the expanded layout, or one source rank's block of the rank layout, the order in which rows land
is the scheduler's business.  What is fixed is the multiset of ``(payload, scales, weight, routing row)`` records
per segment, and that nothing is lost, duplicated or moved across segments.  Alignment padding is unspecified and is
never looked at.  Parity: the reference's result checkers (``tests/utils/checks.py`` there, exercised with injected
faults by ``tests/test_reference.py:119-177``).
"""
from __future__ import annotations

from collections import Counter
from typing import List, Optional, Tuple

import torch

from .reference import RankLayout, XLike


class ResultMismatch(AssertionError):
    """A result violates the dispatch / combine contract; the message names the segment and the kind of damage."""


def _row_bytes(t: Optional[torch.Tensor], rows: torch.Tensor) -> List[bytes]:
    if t is None:
        return [b""] * int(rows.numel())
    picked = t.detach().cpu()[rows].contiguous()
    flat = picked.reshape(picked.shape[0], -1).view(torch.uint8) if picked.numel() else picked.reshape(picked.shape[0], 0)
    return [bytes(r.tolist()) for r in flat]


def _parts(x: XLike) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    return (x[0], x[1]) if isinstance(x, (tuple, list)) else (x, None)


def segments(layout: RankLayout) -> List[Tuple[str, torch.Tensor]]:
    """``(name, row positions)`` of every group of rows whose internal order is free."""
    if layout.expanded:
        return [(f"expert {e}", torch.arange(int(layout.expert_offsets[e]), int(layout.expert_offsets[e] + layout.expert_counts[e])))
                for e in range(layout.num_local_experts)]
    bounds = [0] + torch.cumsum(layout.rank_rows, 0).tolist()
    return [(f"source rank {s}", torch.arange(bounds[s], bounds[s + 1])) for s in range(len(bounds) - 1)]


def check_dispatch(got_x: XLike, got_topk_idx: Optional[torch.Tensor], got_weights: Optional[torch.Tensor],
                   want: Tuple[XLike, Optional[torch.Tensor], Optional[torch.Tensor]], layout: RankLayout) -> None:
    """Raise :class:`ResultMismatch` unless the received rows equal the oracle's ``want`` (one rank's entry of
    ``reference.dispatch``) segment by segment as multisets.  Channels the oracle does not have (no weights, no scales,
    no routing rows in the expanded layout) must be absent from the result as well."""
    (gx, gsf), (wx, wsf) = _parts(got_x), _parts(want[0])
    if int(gx.shape[0]) < layout.num_rows:
        raise ResultMismatch(f"rows: the result holds {int(gx.shape[0])} rows, the layout needs {layout.num_rows}")
    for name, g, w in (("scales", gsf, wsf), ("routing rows", got_topk_idx, want[1]), ("weights", got_weights, want[2])):
        if (g is None) != (w is None):
            raise ResultMismatch(f"{name}: {'missing from' if g is None else 'unexpected in'} the result")
    for name, rows in segments(layout):
        have = Counter(zip(_row_bytes(gx, rows), _row_bytes(gsf, rows), _row_bytes(got_topk_idx, rows), _row_bytes(got_weights, rows)))
        need = Counter(zip(_row_bytes(wx, rows), _row_bytes(wsf, rows), _row_bytes(want[1], rows), _row_bytes(want[2], rows)))
        if have == need:
            continue
        lost, extra = need - have, have - need
        payload_only = Counter(k[0] for k in have.elements()) == Counter(k[0] for k in need.elements())
        kind = "metadata (scales, routing row or weight) of a row differs" if payload_only else \
            f"{sum(lost.values())} expected record(s) missing, {sum(extra.values())} unexpected"
        raise ResultMismatch(f"{name}: {kind}")


def check_combine(got: torch.Tensor, want: torch.Tensor, *, tolerance: float = 0.0) -> None:
    """Raise :class:`ResultMismatch` unless ``got`` equals the oracle's combine output: bit for bit with ``tolerance=0``
    (a combine that adds in the contract's order has one legal answer), else within ``tolerance`` relative to the
    largest expected magnitude (for implementations that are free to reassociate)."""
    if tuple(got.shape) != tuple(want.shape):
        raise ResultMismatch(f"shape: {tuple(got.shape)} instead of {tuple(want.shape)}")
    g, w = got.detach().cpu(), want.detach().cpu()
    if tolerance == 0.0:
        same = (g.contiguous().view(torch.uint8) == w.to(g.dtype).contiguous().view(torch.uint8)).reshape(g.shape[0], -1).all(dim=1) \
            if g.numel() else torch.ones(g.shape[0], dtype=torch.bool)
    else:
        scale = float(w.abs().max()) if w.numel() else 1.0
        same = ((g.double() - w.double()).abs() <= tolerance * max(scale, 1e-30)).reshape(g.shape[0], -1).all(dim=1)
    if not bool(same.all()):
        bad = (~same).nonzero(as_tuple=True)[0]
        raise ResultMismatch(f"token {int(bad[0])}: combined value differs ({int(bad.numel())} of {int(g.shape[0])} tokens)")


__all__ = ["ResultMismatch", "check_combine", "check_dispatch", "segments"]
