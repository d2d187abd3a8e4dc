"""The baseline the native kernels are measured against: expert-parallel MoE from library calls.

* dispatch / combine: ``torch.distributed.all_to_all_single`` with per-rank split sizes (NCCL
  all-to-all-v), one row per (token, slot) -- no rank-level dedup, the usual library formulation;
* experts: bf16 cuBLAS GEMMs per local expert (``torch.matmul``), SwiGLU in eager PyTorch.

Nothing here is used by the product path.  With a world size of 1 the collectives degenerate to
local permutations, which is still the honest single-GPU cost of this formulation.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


@dataclass
class BaselinePlan:
    order: torch.Tensor            # [T * K_valid] permutation that sorts slots by destination expert
    token_of: torch.Tensor         # token of each sorted slot
    slot_weight: torch.Tensor      # routing weight of each sorted slot
    send_counts: List[int]         # rows to each rank
    recv_counts: List[int]         # rows from each rank
    recv_expert_counts: torch.Tensor   # [P, L] rows per (source rank, local expert)
    num_tokens: int


class NcclExpertParallel:
    def __init__(self, group, num_experts: int):
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.num_experts, self.local = num_experts, num_experts // self.world

    def plan(self, topk_idx: torch.Tensor, topk_weights: torch.Tensor) -> BaselinePlan:
        T, K = topk_idx.shape
        flat = topk_idx.reshape(-1)
        valid = (flat >= 0).nonzero(as_tuple=True)[0]
        order = valid[torch.sort(flat[valid], stable=True).indices]
        experts = flat[order]
        counts = torch.bincount(experts, minlength=self.num_experts).view(self.world, self.local)
        if self.world > 1:
            recv = torch.empty_like(counts)
            dist.all_to_all_single(recv, counts, group=self.group)
        else:
            recv = counts.clone()
        send_counts, recv_counts = counts.sum(1).tolist(), recv.sum(1).tolist()       # one host sync, like any a2a-v
        return BaselinePlan(order, torch.div(order, K, rounding_mode="floor"), topk_weights.reshape(-1)[order], send_counts,
                            recv_counts, recv, T)

    def dispatch(self, x: torch.Tensor, plan: BaselinePlan) -> torch.Tensor:
        send = x[plan.token_of]
        if self.world == 1:
            return send
        recv = torch.empty((sum(plan.recv_counts), x.shape[1]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(recv, send, plan.recv_counts, plan.send_counts, group=self.group)
        return recv

    def expert_major(self, rows: torch.Tensor, plan: BaselinePlan) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Received rows are (source, expert)-ordered; regroup them by expert for the GEMMs."""
        counts = plan.recv_expert_counts                      # [P, L]
        expert_of = torch.repeat_interleave(torch.arange(self.local, device=rows.device).repeat(self.world), counts.reshape(-1))
        perm = torch.sort(expert_of, stable=True).indices
        return rows[perm], perm, counts.sum(0)

    def combine(self, rows: torch.Tensor, plan: BaselinePlan, weighted: bool = True) -> torch.Tensor:
        if self.world > 1:
            back = torch.empty((sum(plan.send_counts), rows.shape[1]), dtype=rows.dtype, device=rows.device)
            dist.all_to_all_single(back, rows, plan.send_counts, plan.recv_counts, group=self.group)
        else:
            back = rows
        out = torch.zeros((plan.num_tokens, rows.shape[1]), dtype=torch.float32, device=rows.device)
        vals = back.float() * plan.slot_weight.unsqueeze(1) if weighted else back.float()
        out.index_add_(0, plan.token_of, vals)
        return out.to(torch.bfloat16)


def expert_ffn(rows: torch.Tensor, counts: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """SwiGLU experts on expert-major rows: w1 [L, 2I, H], w2 [L, H, I] bf16; one cuBLAS GEMM pair per expert."""
    out = torch.empty((rows.shape[0], w2.shape[1]), dtype=rows.dtype, device=rows.device)
    start = 0
    for e, c in enumerate(counts.tolist()):
        if c == 0:
            continue
        h = rows[start:start + c] @ w1[e].t()
        gate, up = h.chunk(2, dim=-1)
        out[start:start + c] = (torch.nn.functional.silu(gate) * up) @ w2[e].t()
        start += c
    return out


def moe_forward(ep: NcclExpertParallel, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, w1: torch.Tensor,
                w2: torch.Tensor) -> torch.Tensor:
    plan = ep.plan(topk_idx, topk_weights)
    rows = ep.dispatch(x, plan)
    grouped, perm, counts = ep.expert_major(rows, plan)
    y = expert_ffn(grouped, counts, w1, w2)
    back = torch.empty_like(y)
    back[perm] = y
    return ep.combine(back, plan)
