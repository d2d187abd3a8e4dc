"""Expert-parallel MoE layer for training: autograd through dispatch/combine by handle reversal.

The reference documents the rule (``README.md:168-219``, ``docs/elastic.md:7-17``) but ships no autograd
``Function``: the backward of ``combine`` is a cached ``dispatch`` of the gradient, the backward of
``dispatch`` is a ``combine`` of the row gradients, with the fp32 weight gradients riding the value channel.
"""
from __future__ import annotations


import torch

from ..parallel.elastic import ElasticBuffer


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, buffer: ElasticBuffer, x, topk_idx, topk_weights, num_experts, holder):
        recv_x, _, recv_w, handle, _ = buffer.dispatch(x, topk_idx=topk_idx, topk_weights=topk_weights, num_experts=num_experts,
                                                       do_expand=True)
        ctx.buffer, ctx.handle = buffer, handle
        holder["handle"] = handle
        ctx.mark_non_differentiable(handle.psum_num_recv_tokens_per_expert)
        return recv_x, recv_w, handle.psum_num_recv_tokens_per_expert

    @staticmethod
    def backward(ctx, grad_recv_x, grad_recv_w, _):
        gw = None if grad_recv_w is None else grad_recv_w.float().contiguous()
        if gw is None:
            gw = torch.zeros(grad_recv_x.shape[0], dtype=torch.float32, device=grad_recv_x.device)
        grad_x, grad_w, _ = ctx.buffer.combine(grad_recv_x.to(torch.bfloat16).contiguous(), ctx.handle, topk_weights=gw)
        return None, grad_x, None, grad_w, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, buffer: ElasticBuffer, expert_out, handle):
        out, _, _ = buffer.combine(expert_out, handle)
        ctx.buffer, ctx.handle = buffer, handle
        return out

    @staticmethod
    def backward(ctx, grad_out):
        grad_rows, _, _, _, _ = ctx.buffer.dispatch(grad_out.to(torch.bfloat16).contiguous(), handle=ctx.handle)
        return None, grad_rows, None


class ExpertParallelMoE(torch.nn.Module):
    """SwiGLU experts sharded over the ranks of ``buffer``; forward = dispatch -> local experts -> combine.

    ``w1 [L, 2I, H]`` holds gate rows then up rows, ``w2 [L, H, I]``; both bf16, Kaiming-uniform.
    The routing weight multiplies each expert output row before combine (whose reduction is unweighted).
    """

    def __init__(self, buffer: ElasticBuffer, num_experts: int, hidden: int, intermediate: int, device=None):
        super().__init__()
        self.buffer, self.num_experts = buffer, num_experts
        self.local = num_experts // buffer.world_size
        w1 = torch.empty((self.local, 2 * intermediate, hidden), dtype=torch.bfloat16, device=device)
        w2 = torch.empty((self.local, hidden, intermediate), dtype=torch.bfloat16, device=device)
        for w in (w1, w2):
            for e in range(self.local):
                torch.nn.init.kaiming_uniform_(w[e], a=5 ** 0.5)
        self.w1, self.w2 = torch.nn.Parameter(w1), torch.nn.Parameter(w2)
        self.use_grouped_mm = None        # decided at the first GPU forward (set it to False to force the per-expert loop)

    def experts(self, rows: torch.Tensor, psum: torch.Tensor, counts=None) -> torch.Tensor:
        """SwiGLU experts on expert-major rows.  On a GPU with a usable library grouped GEMM both projections are one
        ``torch._grouped_mm`` each (row ranges from the handle's cumulative counts, which stay on the device);
        otherwise a loop over the experts with the host-side counts of the handle (no device synchronisation)."""
        if rows.is_cuda and self.use_grouped_mm is None:
            from ..utils.grouped_mm import grouped_mm_usable

            self.use_grouped_mm = grouped_mm_usable()
        if rows.is_cuda and self.use_grouped_mm and rows.shape[0] > 0:
            offs = psum.to(torch.int32)
            gate, up = torch._grouped_mm(rows, self.w1.transpose(1, 2), offs=offs).chunk(2, dim=-1)
            return torch._grouped_mm(torch.nn.functional.silu(gate) * up, self.w2.transpose(1, 2), offs=offs)
        bounds = [0]
        for c in (counts if counts is not None else torch.diff(psum, prepend=psum.new_zeros(1)).tolist()):
            bounds.append(bounds[-1] + int(c))
        outs = []
        for e in range(self.local):
            seg = rows[bounds[e]:bounds[e + 1]]
            gate, up = (seg @ self.w1[e].t()).chunk(2, dim=-1)
            outs.append((torch.nn.functional.silu(gate) * up) @ self.w2[e].t())
        return torch.cat(outs, dim=0) if outs else rows.new_zeros((0, self.w2.shape[1]))

    def forward(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        holder = {}
        recv_x, recv_w, psum = _Dispatch.apply(self.buffer, x, topk_idx, topk_weights, self.num_experts, holder)
        y = self.experts(recv_x, psum, holder["handle"].num_recv_tokens_per_expert_list) * recv_w.unsqueeze(1).to(recv_x.dtype)
        return _Combine.apply(self.buffer, y.contiguous(), holder["handle"])


__all__ = ["ExpertParallelMoE"]
