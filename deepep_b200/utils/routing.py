"""Synthetic routing tables shared by the benchmarks and the tests."""
import torch


def group_limited_routes(tokens: int, num_experts: int, topk: int, num_groups: int, topk_groups: int, seed: int = 0,
                         bias_std: float = 0.5) -> torch.Tensor:
    """DeepSeek-V3 gating: pick ``topk_groups`` groups by max score, then ``topk`` experts inside them."""
    g = torch.Generator().manual_seed(seed)
    bias = torch.randn(num_experts, generator=torch.Generator().manual_seed(1234)) * bias_std
    scores = torch.randn((tokens, num_experts), generator=g) + bias
    group_scores = scores.view(tokens, num_groups, -1).amax(dim=-1)
    group_idx = torch.topk(group_scores, topk_groups, dim=-1).indices
    keep = torch.zeros((tokens, num_groups), dtype=torch.bool).scatter_(1, group_idx, True)
    masked = scores.view(tokens, num_groups, -1).masked_fill(~keep.unsqueeze(-1), float("-inf")).view(tokens, num_experts)
    return torch.topk(masked, topk, dim=-1).indices.to(torch.int64)


__all__ = ["group_limited_routes"]
