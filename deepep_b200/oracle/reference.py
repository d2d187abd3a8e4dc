"""All-rank CPU oracle: the semantic definition of dispatch, expansion and combine.

It sees every rank's inputs at once and needs no process group.  The device
kernels and the Gloo engine are checked against it bit for bit.

Ordering and value rules (parity: ``tests/utils/reference.py:39-73`` dispatch,
``:104-131`` combine; dedup rules of ``csrc/kernels/notify/notify.cpp:144-261``):

* ``topk_idx[t, k] < 0`` or ``>= num_experts`` marks an empty slot.
* Expanded layout (``do_expand=True``): one row per (token, slot); rows of a
  destination rank are sorted by (local expert, source rank, source token, slot).
  Every expert's block starts at a multiple of ``expert_alignment``; padding rows are zero.
* Rank layout (``do_expand=False``): one row per (source rank, token) that hits
  the destination, sorted by (source rank, token); ``recv_topk_idx`` holds
  destination-local expert ids and -1 elsewhere.
* High-throughput combine: rows of one (source token, destination rank) are
  summed in slot order in fp32 and rounded to bf16 (the partial that crosses
  NVLink); the source sums the partials in destination-rank order in fp32,
  adds the optional biases, and rounds to bf16.  Weights travel on an
  independent fp32 channel and never scale the payload.
* Low-latency combine: ``sum_k w_k * row_k`` in slot order in fp32, one rounding.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple, Union

import torch

from ..utils.math import per_token_cast_to_fp8

Tensor = torch.Tensor
XLike = Union[Tensor, Tuple[Tensor, Tensor]]


@dataclass
class RankLayout:
    """Everything one destination rank knows after notify."""
    expanded: bool
    num_local_experts: int
    expert_alignment: int
    row_source: Tensor            # [R] source rank of each valid row
    row_token: Tensor             # [R] token index on the source
    row_slot: Tensor              # [R] top-k slot (expanded) or -1
    row_index: Tensor             # [R] position of each valid row in the (padded) output
    num_rows: int                 # output rows including alignment padding
    expert_counts: Tensor         # [L] unaligned rows per local expert (slots, not unique tokens)
    expert_offsets: Tensor        # [L + 1] aligned exclusive prefix
    rank_rows: Tensor             # [P] rank-layout rows (unique tokens) received from each source
    recv_topk_idx: Optional[Tensor] = None      # rank layout only: [R, K] local ids
    slot_hits: Optional[Tensor] = None          # rank layout only: [R, K] bool


def _valid(topk_idx: Tensor, num_experts: int) -> Tensor:
    return (topk_idx >= 0) & (topk_idx < num_experts)


def build_layouts(topk_idx: Sequence[Tensor], num_experts: int, *, do_expand: bool = True,
                  expert_alignment: int = 1) -> List[RankLayout]:
    world = len(topk_idx)
    assert num_experts % world == 0, "num_experts must be divisible by the world size"
    local = num_experts // world
    k = topk_idx[0].shape[1]
    layouts = []
    for dst in range(world):
        srcs, toks, slots, exps, rank_rows = [], [], [], [], []
        tok_rows_src, tok_rows_tok, tok_rows_idx, tok_rows_hit = [], [], [], []
        for src, idx in enumerate(topk_idx):
            idx = idx.long()
            hit = _valid(idx, num_experts) & (torch.div(idx, local, rounding_mode="floor") == dst)
            t_ids, s_ids = hit.nonzero(as_tuple=True)  # row-major: (token, slot) ascending
            srcs.append(torch.full_like(t_ids, src))
            toks.append(t_ids)
            slots.append(s_ids)
            exps.append(idx[t_ids, s_ids] - dst * local)
            tok_hit = hit.any(dim=1).nonzero(as_tuple=True)[0]
            rank_rows.append(tok_hit.numel())
            tok_rows_src.append(torch.full_like(tok_hit, src))
            tok_rows_tok.append(tok_hit)
            tok_rows_idx.append(torch.where(hit[tok_hit], idx[tok_hit] - dst * local, torch.full_like(idx[tok_hit], -1)))
            tok_rows_hit.append(hit[tok_hit])
        src_all, tok_all, slot_all, exp_all = map(torch.cat, (srcs, toks, slots, exps))
        counts = torch.bincount(exp_all, minlength=local)[:local] if exp_all.numel() else torch.zeros(local, dtype=torch.long)
        aligned = (counts + expert_alignment - 1) // expert_alignment * expert_alignment
        offsets = torch.zeros(local + 1, dtype=torch.long)
        offsets[1:] = torch.cumsum(aligned, 0)
        if do_expand:
            order = torch.sort(exp_all, stable=True).indices  # ties keep (source, token, slot) order
            src_o, tok_o, slot_o, exp_o = src_all[order], tok_all[order], slot_all[order], exp_all[order]
            unaligned_start = torch.zeros(local + 1, dtype=torch.long)
            unaligned_start[1:] = torch.cumsum(counts, 0)
            within = torch.arange(exp_o.numel()) - unaligned_start[exp_o]
            layouts.append(RankLayout(True, local, expert_alignment, src_o, tok_o, slot_o, offsets[exp_o] + within,
                                      int(offsets[-1]), counts, offsets, torch.tensor(rank_rows)))
        else:
            src_r, tok_r = torch.cat(tok_rows_src), torch.cat(tok_rows_tok)
            idx_r = torch.cat(tok_rows_idx) if tok_rows_idx else torch.zeros((0, k), dtype=torch.long)
            hit_r = torch.cat(tok_rows_hit) if tok_rows_hit else torch.zeros((0, k), dtype=torch.bool)
            layouts.append(RankLayout(False, local, expert_alignment, src_r, tok_r, torch.full_like(src_r, -1),
                                      torch.arange(src_r.numel()), src_r.numel(), counts, offsets,
                                      torch.tensor(rank_rows), idx_r, hit_r))
    return layouts


def _split(x: XLike):
    return (x[0], x[1]) if isinstance(x, (tuple, list)) else (x, None)


def dispatch(xs: Sequence[XLike], topk_idx: Sequence[Tensor], topk_weights: Optional[Sequence[Tensor]],
             num_experts: int, *, do_expand: bool = True, expert_alignment: int = 1,
             quantize_fp8: bool = False, layouts: Optional[List[RankLayout]] = None):
    """Return (per-rank list of (recv_x, recv_topk_idx, recv_topk_weights), layouts)."""
    if quantize_fp8:
        xs = [per_token_cast_to_fp8(x) for x in xs]
    layouts = layouts or build_layouts(topk_idx, num_experts, do_expand=do_expand, expert_alignment=expert_alignment)
    outs = []
    for lay in layouts:
        data0, sf0 = _split(xs[0])
        recv = torch.zeros((lay.num_rows, data0.shape[1]), dtype=data0.dtype)
        recv_sf = None if sf0 is None else torch.zeros((lay.num_rows, sf0.shape[1]), dtype=sf0.dtype)
        if lay.expanded:
            recv_w = None if topk_weights is None else torch.zeros(lay.num_rows, dtype=torch.float32)
        else:
            recv_w = None if topk_weights is None else torch.zeros((lay.num_rows, topk_idx[0].shape[1]), dtype=torch.float32)
        for src in range(len(xs)):
            sel = (lay.row_source == src).nonzero(as_tuple=True)[0]
            if sel.numel() == 0:
                continue
            data, sf = _split(xs[src])
            rows, toks = lay.row_index[sel], lay.row_token[sel]
            recv[rows] = data[toks]
            if sf is not None:
                recv_sf[rows] = sf[toks]
            if recv_w is not None:
                w = topk_weights[src].float()
                if lay.expanded:
                    recv_w[rows] = w[toks, lay.row_slot[sel]]
                else:
                    recv_w[rows] = torch.where(lay.slot_hits[sel], w[toks], torch.zeros_like(w[toks]))
        out_x = recv if recv_sf is None else (recv, recv_sf)
        outs.append((out_x, None if lay.expanded else lay.recv_topk_idx, recv_w))
    return outs, layouts


def combine(expert_out: Sequence[Tensor], layouts: List[RankLayout], num_tokens: Sequence[int], num_topk: int,
            *, topk_weights: Optional[Sequence[Tensor]] = None,
            bias: Optional[Sequence[Union[Tensor, Tuple[Tensor, Tensor], None]]] = None):
    """High-throughput combine. Returns per-source (combined_x bf16 [T, H], combined_w fp32 [T, K] | None)."""
    world = len(layouts)
    hidden = expert_out[0].shape[1]
    partial = [torch.zeros((n, world, hidden), dtype=torch.float32) for n in num_tokens]
    wout = None if topk_weights is None else [torch.zeros((n, num_topk), dtype=torch.float32) for n in num_tokens]
    for dst, lay in enumerate(layouts):
        rows_x = expert_out[dst].float()
        if lay.expanded:
            for slot in range(num_topk):  # slot order fixes the fp32 summation order
                sel = (lay.row_slot == slot).nonzero(as_tuple=True)[0]
                for src in range(world):
                    s2 = sel[lay.row_source[sel] == src]
                    if s2.numel():
                        partial[src][lay.row_token[s2], dst] += rows_x[lay.row_index[s2]]
                        if wout is not None:
                            wout[src][lay.row_token[s2], slot] = topk_weights[dst].float()[lay.row_index[s2]]
        else:
            for src in range(world):
                sel = (lay.row_source == src).nonzero(as_tuple=True)[0]
                if sel.numel():
                    partial[src][lay.row_token[sel], dst] += rows_x[lay.row_index[sel]]
                    if wout is not None:
                        w = topk_weights[dst].float()[lay.row_index[sel]]
                        cur = wout[src][lay.row_token[sel]]
                        wout[src][lay.row_token[sel]] = torch.where(lay.slot_hits[sel], w, cur)
    outs = []
    for src in range(world):
        p16 = partial[src].to(torch.bfloat16).float()  # the partial crosses the link as bf16
        acc = torch.zeros((num_tokens[src], hidden), dtype=torch.float32)
        for dst in range(world):
            acc += p16[:, dst]
        if bias is not None and bias[src] is not None:
            for b in (bias[src] if isinstance(bias[src], (tuple, list)) else (bias[src],)):
                if b is not None:
                    acc += b.float()
        outs.append((acc.to(torch.bfloat16), None if wout is None else wout[src]))
    return outs


def low_latency_combine(expert_out: Sequence[Tensor], layouts: List[RankLayout], topk_weights: Sequence[Tensor],
                        num_tokens: Sequence[int]):
    """``sum_k w_k * row_k`` in slot order, fp32 accumulate, bf16 result, per source rank."""
    world, hidden = len(layouts), expert_out[0].shape[1]
    k = topk_weights[0].shape[1]
    acc = [torch.zeros((n, hidden), dtype=torch.float32) for n in num_tokens]
    for slot in range(k):
        for dst, lay in enumerate(layouts):
            assert lay.expanded
            sel = (lay.row_slot == slot).nonzero(as_tuple=True)[0]
            for src in range(world):
                s2 = sel[lay.row_source[sel] == src]
                if s2.numel():
                    toks = lay.row_token[s2]
                    w = topk_weights[src].float()[toks, slot].unsqueeze(1)
                    acc[src][toks] += w * expert_out[dst].float()[lay.row_index[s2]]
    return [a.to(torch.bfloat16) for a in acc]


def expected_roundtrip(xs: Sequence[Tensor], topk_idx: Sequence[Tensor], topk_weights: Sequence[Tensor], num_experts: int):
    """Source-side answer of dispatch -> (row * weight) -> combine computed without any layout: sum_k w_k x."""
    outs = []
    for x, idx, w in zip(xs, topk_idx, topk_weights):
        ok = _valid(idx.long(), num_experts).float()
        outs.append((x.float() * (w.float() * ok).sum(dim=1, keepdim=True)))
    return outs


__all__ = ["RankLayout", "build_layouts", "combine", "dispatch", "expected_roundtrip", "low_latency_combine"]
