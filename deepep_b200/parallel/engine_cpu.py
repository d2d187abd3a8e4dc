"""CPU engine: the same operations over a host process group (Gloo) or a single process.

Every rank all-gathers the small routing tables and the payload through the
control plane and evaluates the all-rank oracle for its own rank.  It defines
the behaviour the CUDA engine must reproduce bit for bit, and lets the whole
Python orchestration (handles, events, backward by handle reversal) run on
machines without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..oracle import reference as R


@dataclass
class CpuPlan:
    num_tokens: int
    num_experts: int
    num_topk: int
    expand: bool
    alignment: int
    num_rows: int
    num_staged_rows: int
    expert_counts_list: List[int]
    topk_idx: torch.Tensor
    layouts: list                       # every rank's RankLayout
    all_tokens: List[int]
    all_idx: List[torch.Tensor]
    all_w: Optional[List[torch.Tensor]]
    expert_counts: torch.Tensor
    expert_offsets: torch.Tensor
    rank_rows: torch.Tensor
    recv_row_src: torch.Tensor
    recv_w: Optional[torch.Tensor]
    recv_idx: Optional[torch.Tensor]
    slot_row: Optional[torch.Tensor] = None
    send_slot: Optional[torch.Tensor] = None
    stage_meta: Optional[torch.Tensor] = None
    chunk_start: Optional[torch.Tensor] = None
    has_weights: bool = False
    low_latency: bool = False
    rank_matrix: Optional[torch.Tensor] = None
    send_chunk_prefix: Optional[torch.Tensor] = None
    exact_rows: int = 0                 # rows that carry data; ``num_rows`` is larger when the counts were not read back

    def tensors(self):
        return [t for t in (self.topk_idx, self.expert_counts, self.expert_offsets, self.recv_row_src, self.recv_w,
                            self.recv_idx) if t is not None]


class CpuEngine:
    def __init__(self, control, max_tokens: int, hidden: int, topk: int):
        self.control, self.rank, self.world = control, control.rank, control.size
        self.max_tokens, self.hidden, self.topk = max_tokens, hidden, topk
        self.n = 1

    def check_status(self) -> None:
        pass

    def _gather(self, obj):
        return self.control.all_gather_object(obj)

    def notify(self, topk_idx: Sequence[torch.Tensor], topk_w: Sequence[Optional[torch.Tensor]], num_experts: int,
               expand: bool = True, alignment: int = 1, cpu_sync: bool = True, blocks: int = 0, stream=None,
               rank_matrix: bool = False) -> List[CpuPlan]:
        del blocks, stream
        idx = topk_idx[0].cpu().long()
        w = None if topk_w[0] is None else topk_w[0].cpu().float()
        gathered = self._gather((idx, w))
        all_idx = [g[0] for g in gathered]
        all_w = None if any(g[1] is None for g in gathered) else [g[1] for g in gathered]
        layouts = R.build_layouts(all_idx, num_experts, do_expand=expand, expert_alignment=alignment)
        lay = layouts[self.rank]
        k = idx.shape[1]
        src = torch.full((lay.num_rows,), -1, dtype=torch.int32)
        slot = lay.row_slot.clamp(min=0)
        src[lay.row_index] = ((lay.row_source * self.max_tokens + lay.row_token) * k + slot).int()
        recv_w = None
        if all_w is not None:
            fake_x = [torch.zeros((i.shape[0], 1)) for i in all_idx]
            outs, _ = R.dispatch(fake_x, all_idx, all_w, num_experts, do_expand=expand, layouts=layouts)
            recv_w = outs[self.rank][2]
        rank_rows = torch.zeros(self.world + 1, dtype=torch.int32)
        rank_rows[1:] = torch.cumsum(lay.rank_rows, 0).int()
        plan = CpuPlan(idx.shape[0], num_experts, k, expand, alignment, lay.num_rows, int(rank_rows[-1]),
                       lay.expert_counts.tolist(), topk_idx[0], layouts, [i.shape[0] for i in all_idx], all_idx, all_w,
                       lay.expert_counts.int(), lay.expert_offsets.int(), rank_rows, src, recv_w,
                       lay.recv_topk_idx, has_weights=all_w is not None)
        plan.exact_rows = lay.num_rows
        if not cpu_sync:
            # No read-back of the counts: like the CUDA engine, hand out the worst-case number of rows (the rows past the
            # real count carry no data) and no per-expert list.
            local = num_experts // self.world
            capacity = self.world * self.max_tokens * (min(k, local) if expand else 1)
            if expand and alignment > 1:
                capacity += local * (alignment - 1)
            extra = capacity - lay.num_rows
            plan.num_rows, plan.expert_counts_list = capacity, None
            plan.recv_row_src = torch.cat([src, torch.full((extra,), -1, dtype=torch.int32)])
            if plan.recv_w is not None:
                plan.recv_w = torch.cat([plan.recv_w, plan.recv_w.new_zeros((extra,) + tuple(plan.recv_w.shape[1:]))])
            if plan.recv_idx is not None:
                plan.recv_idx = torch.cat([plan.recv_idx, plan.recv_idx.new_full((extra, k), -1)])
        if rank_matrix:     # what the V1 handle is built from (the CUDA engine gets these from the layout kernel)
            local, chunk = num_experts // self.world, 64
            hits = []
            for i in all_idx:
                ok = (i >= 0) & (i < num_experts)
                dst = torch.where(ok, torch.div(i.clamp(min=0), local, rounding_mode="floor"), torch.full_like(i, -1))
                hits.append(torch.stack([(dst == d).any(dim=1) for d in range(self.world)], dim=1))      # [T_r, P]
            plan.rank_matrix = torch.stack([h.sum(0) for h in hits]).int()
            mine = hits[self.rank]
            pos = torch.cumsum(mine.int(), 0) - 1
            plan.send_slot = torch.where(mine, pos, torch.full_like(pos, -1)).int()
            tiles = max(1, -(-idx.shape[0] // chunk))
            pad = torch.zeros((tiles * chunk, self.world), dtype=torch.int64)
            pad[:mine.shape[0]] = mine
            per_chunk = pad.view(tiles, chunk, self.world).sum(1)                                        # [tiles, P]
            plan.send_chunk_prefix = (torch.cumsum(per_chunk, 0) - per_chunk).t().contiguous().int()     # exclusive, [P, tiles]
            nt = -(-self.max_tokens // chunk)
            starts = torch.zeros((self.world, nt + 1), dtype=torch.int32)
            for r, h in enumerate(hits):
                col = torch.zeros(nt * chunk, dtype=torch.int64)
                col[:h.shape[0]] = h[:, self.rank]
                starts[r, 1:] = torch.cumsum(col.view(nt, chunk).sum(1), 0).int()
            plan.chunk_start = starts
        return [plan]

    def dispatch(self, xs: Sequence, plans: Sequence[CpuPlan], mode: int, blocks: int = 0, stream=None):
        del blocks, stream
        plan = plans[0]
        x = xs[0]
        x = tuple(t.cpu() for t in x) if isinstance(x, (tuple, list)) else x.cpu()
        if isinstance(x, tuple):     # e4m3 tensors do not survive the object pickling of the control plane: send their bytes
            all_x = [(codes.view(torch.float8_e4m3fn), sf) for codes, sf in self._gather((x[0].view(torch.uint8), x[1]))]
        else:
            all_x = self._gather(x)
        outs, _ = R.dispatch(all_x, plan.all_idx, None, plan.num_experts, do_expand=plan.expand,
                             quantize_fp8=(mode == 2), layouts=plan.layouts)
        out = outs[self.rank][0]
        data, sf = (out[0], out[1]) if isinstance(out, tuple) else (out, None)
        extra = plan.num_rows - data.shape[0]
        if extra > 0:           # worst-case outputs: rows past the real count are zero
            data = torch.cat([data, data.new_zeros((extra, data.shape[1]))])
            sf = None if sf is None else torch.cat([sf, sf.new_zeros((extra, sf.shape[1]))])
        return [(data, sf)]

    def combine(self, xs: Sequence[torch.Tensor], plans: Sequence[CpuPlan], ws: Sequence[Optional[torch.Tensor]],
                bias: Sequence = None, blocks: int = 0, stream=None):
        del blocks, stream
        plan = plans[0]
        rows = plan.exact_rows or plan.num_rows
        gathered = self._gather((xs[0].cpu()[:rows], None if ws[0] is None else ws[0].cpu().float()[:rows],
                                 None if bias is None else bias[0]))
        all_x = [g[0] for g in gathered]
        all_w = None if any(g[1] is None for g in gathered) else [g[1] for g in gathered]
        all_b = None if bias is None else [g[2] for g in gathered]
        outs = R.combine(all_x, plan.layouts, plan.all_tokens, plan.num_topk, topk_weights=all_w, bias=all_b)
        return [outs[self.rank]]

    def ll_combine(self, xs: Sequence[torch.Tensor], plans: Sequence[CpuPlan], stream=None):
        plan = plans[0]
        all_x = self._gather(xs[0].cpu()[:plan.exact_rows or plan.num_rows])
        return [R.low_latency_combine(all_x, plan.layouts, plan.all_w, plan.all_tokens)[self.rank]]

    def barrier(self, stream=None) -> None:
        self.control.barrier()
