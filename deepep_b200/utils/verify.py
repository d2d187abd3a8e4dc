"""Self-checks of a live buffer that need no all-rank oracle run: every rank verifies what it received against small
facts gathered from the other ranks (row checksums, routing tables), so the checks scale to the benchmark shapes.

``verify_dispatch_combine`` covers the high-throughput path (expanded layout), ``verify_low_latency`` the decode
path.  Both are collective, return ``(ok, details)`` with ``ok`` agreed by all ranks, and compare bit for bit:
the facts restate the ordering and numeric contracts of the reference (rows sorted by (local expert, source rank,
source token, slot), ``tests/utils/reference.py:39-73``; fp32 sum -> bf16 partial per expert rank -> fp32 sum in
rank order, ``docs/elastic.md:69-72``; low latency ``sum_k w_k * row_k``, ``docs/elastic.md:101-104``).
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch


def row_checksums(x: torch.Tensor) -> torch.Tensor:
    """Two 64-bit sums per row over the raw 16-bit (or 8-bit) codes: a plain one and a position-weighted one."""
    codes = x.contiguous().view(torch.int16 if x.element_size() == 2 else torch.int8).to(torch.int64)
    weight = (torch.arange(codes.shape[1], device=x.device, dtype=torch.int64) % 251) + 1
    return torch.stack((codes.sum(1), (codes * weight).sum(1)), dim=1)


def _lookup(tables: List[torch.Tensor], s: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
    """``tables[s[i]][t[i]]`` for every i: the per-rank tables are stacked once and indexed by a global row number."""
    sizes = torch.tensor([0] + [tab.shape[0] for tab in tables])
    return torch.cat(tables)[torch.cumsum(sizes, 0)[s] + t]


def _agree(buf, ok: bool) -> bool:
    return all(buf.control.all_gather_object(bool(ok)))


def _first_valid(idx: torch.Tensor, num_experts: int) -> torch.Tensor:
    """[T, K] bool: the slot names an expert in range that no earlier slot of the row names."""
    valid = (idx >= 0) & (idx < num_experts)
    same = idx.unsqueeze(2) == idx.unsqueeze(1)                       # [T, K, K]
    earlier = torch.tril(torch.ones(idx.shape[1], idx.shape[1], dtype=torch.bool, device=idx.device), diagonal=-1)
    return valid & ~(same & earlier & valid.unsqueeze(1)).any(dim=2)


def verify_dispatch_combine(buf, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, num_experts: int
                            ) -> Tuple[bool, Dict]:
    """One fresh dispatch (expanded layout) and one combine with identity experts, checked on every rank."""
    rank, world, tmax = buf.rank, buf.world_size, buf.num_max_tokens_per_rank
    K, local = topk_idx.shape[1], num_experts // world
    recv_x, _, recv_w, handle, _ = buf.dispatch(x, topk_idx=topk_idx, topk_weights=topk_weights, num_experts=num_experts,
                                                do_expand=True)
    facts = buf.control.all_gather_object((row_checksums(x).cpu(), topk_idx.cpu(), topk_weights.cpu()))
    all_idx = [f[1] for f in facts]
    details: Dict = {}
    rows = recv_x.shape[0]
    counts = list(handle.num_recv_tokens_per_expert_list)
    src = handle.recv_src_metadata[:rows].cpu().long()
    s, t, k = src // (tmax * K), (src // K) % tmax, src % K
    # (1) every routed (source, token, slot) of this rank's experts appears exactly once, expert-major and sorted inside an expert
    expected = 0
    for r, idx in enumerate(all_idx):
        mine = _first_valid(idx, num_experts) & (torch.div(idx.clamp(min=0), local, rounding_mode="floor") == rank)
        expected += int(mine.sum())
    ok_count = rows == expected == sum(counts) and len(counts) == local
    expert_of_row = torch.repeat_interleave(torch.arange(local), torch.tensor(counts)) + rank * local
    ok_range = bool(((s >= 0) & (s < world)).all()) and all(bool((t[s == r] < all_idx[r].shape[0]).all()) for r in range(world))
    if not (ok_count and ok_range):
        return _agree(buf, False), dict(rows=rows, expected_rows=expected, counts_ok=ok_count, sources_in_range=ok_range)
    named = _lookup(all_idx, s, t).gather(1, k.unsqueeze(1)).squeeze(1)
    ok_expert = bool(torch.equal(named, expert_of_row))
    same_expert = expert_of_row[1:] == expert_of_row[:-1]
    ok_order = bool(((src[1:] > src[:-1]) | ~same_expert).all()) if rows > 1 else True
    # (2) payload and weights of every row are those of its source token
    sums = row_checksums(recv_x).cpu()
    ok_payload = bool(torch.equal(sums, _lookup([f[0] for f in facts], s, t)))
    want_w = _lookup([f[2] for f in facts], s, t).gather(1, k.unsqueeze(1)).squeeze(1)
    ok_weights = bool(torch.equal(recv_w.cpu(), want_w))
    # (3) combine with identity experts: out[t] = bf16(sum over ranks d of bf16(n_d * x[t])), n_d = distinct experts of t on d
    combined, _, _ = buf.combine(recv_x, handle)
    first = _first_valid(topk_idx, num_experts)
    dst = torch.div(topk_idx.clamp(min=0), local, rounding_mode="floor")
    acc = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    for d in range(world):
        n_d = (first & (dst == d)).sum(dim=1, keepdim=True).float()
        acc += (x.float() * n_d).bfloat16().float()        # n_d * x is exact in fp32 (a sum of n_d equal bf16 values)
    ok_combine = bool(torch.equal(combined.view(torch.int16), acc.bfloat16().view(torch.int16)))
    details.update(rows=rows, counts_ok=ok_count, experts_ok=ok_expert, order_ok=ok_order, payload_ok=ok_payload,
                   weights_ok=ok_weights, combine_ok=ok_combine)
    ok = _agree(buf, ok_count and ok_expert and ok_order and ok_payload and ok_weights and ok_combine)
    return ok, details


def verify_low_latency(buf, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, num_experts: int
                       ) -> Tuple[bool, Dict]:
    """One low-latency dispatch (bf16, or fp8 when the buffer quantises) and one combine whose expert outputs are the
    source rows themselves: ``out[t] = sum_k w[t, k] * x[t]`` in slot order, separate fp32 multiply and add."""
    from .math import per_token_cast_to_fp8

    rank, world, tmax = buf.rank, buf.world_size, buf.num_max_tokens_per_rank
    K, local = topk_idx.shape[1], num_experts // world
    out_x, _, recv_w, handle, _ = buf.dispatch(x, topk_idx=topk_idx, topk_weights=topk_weights, num_experts=num_experts)
    if not handle.is_low_latency:
        return _agree(buf, False), {"error": "the buffer did not take the low-latency path"}
    facts = buf.control.all_gather_object((x.cpu(), topk_idx.cpu(), topk_weights.cpu()))
    fp8 = isinstance(out_x, (tuple, list))
    recv_x = out_x[0] if fp8 else out_x
    rows = recv_x.shape[0]
    src = handle.recv_src_metadata[:rows].cpu().long()
    s, t, k = src // (tmax * K), (src // K) % tmax, src % K
    src_rows = _lookup([f[0] for f in facts], s, t)
    mismatch = {}
    if fp8:
        q, sf = per_token_cast_to_fp8(src_rows)          # the recipe, evaluated on the host like the oracle does
        bad_q = int((recv_x.cpu().view(torch.int8) != q.view(torch.int8)).sum())
        bad_sf = int((out_x[1].cpu() != sf).sum())
        ok_payload = bad_q == 0 and bad_sf == 0
        mismatch = dict(code_mismatches=bad_q, scale_mismatches=bad_sf)
    else:
        ok_payload = bool(torch.equal(recv_x.cpu().view(torch.int16), src_rows.view(torch.int16)))
    named = _lookup([f[1] for f in facts], s, t).gather(1, k.unsqueeze(1)).squeeze(1)
    counts = list(handle.num_recv_tokens_per_expert_list)
    expert_of_row = torch.repeat_interleave(torch.arange(local), torch.tensor(counts)) + rank * local
    ok_expert = sum(counts) == rows and bool(torch.equal(named, expert_of_row))
    combined, _, _ = buf.combine(src_rows.to(x.device), handle)
    first = _first_valid(topk_idx, num_experts)
    acc = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    xf = x.float()
    for slot in range(K):
        term = topk_weights[:, slot:slot + 1].float() * xf
        acc = torch.where(first[:, slot:slot + 1], acc + term, acc)
    ok_combine = bool(torch.equal(combined.view(torch.int16), acc.bfloat16().view(torch.int16)))
    details = dict(rows=rows, payload_ok=ok_payload, experts_ok=ok_expert, combine_ok=ok_combine, fp8=fp8, **mismatch)
    return _agree(buf, ok_payload and ok_expert and ok_combine), details


__all__ = ["row_checksums", "verify_dispatch_combine", "verify_low_latency"]
