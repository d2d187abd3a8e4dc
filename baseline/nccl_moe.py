"""The baseline the native kernels are measured against: expert-parallel MoE from library calls.

* dispatch / combine: ``torch.distributed.all_to_all_single`` with per-rank split sizes (NCCL all-to-all-v) and
  rank-level dedup: a token crosses the link once per destination rank and is expanded to that rank's experts by a
  local gather; the way back pre-reduces a token's rows on the expert rank (fp32 accumulate, bf16 on the wire) and
  reduces the per-rank partials at the source.  Every index tensor and split size is computed once in ``plan`` --
  nothing inside ``dispatch`` / ``combine`` / ``moe_forward`` synchronises with the host.
* experts: one grouped GEMM per projection over expert-major rows (``torch._grouped_mm``, bf16), SwiGLU in eager
  PyTorch.  If the grouped kernel is missing or does not run on this device (``select_gemm`` probes it in a child
  process), a per-expert ``torch.matmul`` (cuBLAS) loop over host-side counts is used.  There is no fp8 variant: the
  row-wise scaled grouped GEMM of this PyTorch build is compiled for another architecture and aborts on sm_100.

Nothing here is used by the product path.  With a world size of 1 the collectives degenerate to local copies,
which is still the honest single-GPU cost of this formulation.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class BaselinePlan:
    num_tokens: int
    send_token: torch.Tensor           # [S] source token of every sent row, sorted by destination rank
    send_counts: List[int]             # rows to each rank
    recv_counts: List[int]             # rows from each rank
    expand_from: torch.Tensor          # [R] received row that feeds every expert-major row
    expert_offsets: torch.Tensor       # int32 [L] cumulative row ends of the local experts (grouped-GEMM offsets)
    expert_counts: List[int]           # rows per local expert (host copy, for the fallback loop)
    row_weight: torch.Tensor           # fp32 [R] routing weight of every expert-major row
    num_recv: int


class NcclExpertParallel:
    def __init__(self, group, num_experts: int):
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.num_experts, self.local = num_experts, num_experts // self.world

    def _a2a(self, send: torch.Tensor, send_counts: List[int], recv_counts: List[int]) -> torch.Tensor:
        if self.world == 1:
            return send
        recv = torch.empty((sum(recv_counts),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        dist.all_to_all_single(recv, send, recv_counts, send_counts, group=self.group)
        return recv

    def plan(self, topk_idx: torch.Tensor, topk_weights: torch.Tensor) -> BaselinePlan:
        """Routing metadata of one batch.  Host synchronisation happens here, once, never in the per-step calls."""
        T, K = topk_idx.shape
        dev = topk_idx.device
        valid = topk_idx >= 0
        dst = torch.where(valid, torch.div(topk_idx, self.local, rounding_mode="floor"), torch.full_like(topk_idx, -1))
        hit = (dst.unsqueeze(-1) == torch.arange(self.world, device=dev)).any(dim=1)        # [T, P]
        pairs = hit.t().nonzero()                                  # (rank, token), sorted by rank then token
        send_token = pairs[:, 1].contiguous()
        send_counts = hit.sum(0).tolist()
        if self.world > 1:
            counts_dev = torch.tensor(send_counts, device=dev)
            recv_dev = torch.empty_like(counts_dev)
            dist.all_to_all_single(recv_dev, counts_dev, group=self.group)
            recv_counts = recv_dev.tolist()
        else:
            recv_counts = list(send_counts)
        # the receivers need the routing rows of the tokens they get
        recv_idx = self._a2a(topk_idx[send_token].contiguous(), send_counts, recv_counts)
        recv_w = self._a2a(topk_weights[send_token].float().contiguous(), send_counts, recv_counts)
        mine = (recv_idx >= self.rank * self.local) & (recv_idx < (self.rank + 1) * self.local)
        rows, slots = mine.nonzero(as_tuple=True)
        local_expert = recv_idx[rows, slots] - self.rank * self.local
        order = torch.sort(local_expert, stable=True).indices       # expert-major, (source, token, slot) inside an expert
        counts = torch.bincount(local_expert, minlength=self.local)
        return BaselinePlan(T, send_token, send_counts, recv_counts, rows[order].contiguous(),
                            torch.cumsum(counts, 0).to(torch.int32), counts.tolist(), recv_w[rows, slots][order].contiguous(),
                            int(recv_idx.shape[0]))

    def dispatch(self, x: torch.Tensor, plan: BaselinePlan) -> torch.Tensor:
        """[T, H] -> expert-major rows [R, H] of this rank's experts."""
        return self._a2a(x[plan.send_token], plan.send_counts, plan.recv_counts)[plan.expand_from]

    def combine(self, rows: torch.Tensor, plan: BaselinePlan, weighted: bool = True) -> torch.Tensor:
        """Expert-major rows [R, H] -> [T, H] bf16; fp32 accumulation, one bf16 partial per (token, rank) on the wire."""
        vals = rows.float() * plan.row_weight.unsqueeze(1) if weighted else rows.float()
        partial = torch.zeros((plan.num_recv, rows.shape[1]), dtype=torch.float32, device=rows.device)
        partial.index_add_(0, plan.expand_from, vals)
        back = self._a2a(partial.to(torch.bfloat16), plan.recv_counts, plan.send_counts)
        out = torch.zeros((plan.num_tokens, rows.shape[1]), dtype=torch.float32, device=rows.device)
        out.index_add_(0, plan.send_token, back.float())
        return out.to(torch.bfloat16)


_grouped_ok: Optional[bool] = False      # set by select_gemm(); the per-expert loop until then


def _grouped_mm(rows: torch.Tensor, weight_t: torch.Tensor, plan: BaselinePlan) -> torch.Tensor:
    """rows [R, K] bf16 x weight_t [L, K, N] bf16 -> [R, N]; expert e owns rows offsets[e-1]..offsets[e]."""
    if _grouped_ok:
        return torch._grouped_mm(rows, weight_t, offs=plan.expert_offsets)
    out = torch.empty((rows.shape[0], weight_t.shape[2]), dtype=rows.dtype, device=rows.device)
    start = 0
    for e, c in enumerate(plan.expert_counts):
        if c:
            torch.matmul(rows[start:start + c], weight_t[e], out=out[start:start + c])
        start += c
    return out


class ExpertWeights:
    """SwiGLU expert weights in the layouts the library GEMMs want: w1 [L, 2I, H], w2 [L, H, I] bf16."""

    def __init__(self, w1: torch.Tensor, w2: torch.Tensor):
        self.w1_t, self.w2_t = w1.transpose(1, 2), w2.transpose(1, 2)          # [L, K, N] views, K-major memory


def expert_ffn(rows: torch.Tensor, plan: BaselinePlan, weights: ExpertWeights) -> torch.Tensor:
    """SwiGLU experts on expert-major rows."""
    gate, up = _grouped_mm(rows, weights.w1_t, plan).chunk(2, dim=-1)
    return _grouped_mm(torch.nn.functional.silu(gate) * up, weights.w2_t, plan)


def moe_forward(ep: NcclExpertParallel, x: torch.Tensor, plan: BaselinePlan, weights: ExpertWeights) -> torch.Tensor:
    """One MoE layer from a prepared plan: dispatch -> grouped SwiGLU experts -> weighted combine."""
    return ep.combine(expert_ffn(ep.dispatch(x, plan), plan, weights), plan, weighted=True)


def select_gemm(use_grouped: Optional[bool] = None) -> bool:
    """Chooses between the library's grouped GEMM and the per-expert loop; returns whether the grouped one is used.

    ``None`` probes ``torch._grouped_mm`` in a child process (a library kernel built for another architecture aborts the
    process that launches it, which must not be the benchmark itself); the caller passes the result to the other ranks."""
    global _grouped_ok
    from deepep_b200.utils.grouped_mm import grouped_mm_usable

    _grouped_ok = grouped_mm_usable(use_grouped)
    return _grouped_ok
