"""Route generators and comparison helpers shared by CPU and GPU tests.

Route modes follow the reference's device tests (``tests/elastic/test_dispatch.py:254``):
normal, random, invalid (-1 slots), empty (all -1 rows), hotspot (one hot expert),
plus DeepSeek-V3 group-limited gating for the benchmark shapes.
"""
import torch


def make_routes(mode: str, tokens: int, num_experts: int, topk: int, world: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    scores = torch.rand((tokens, num_experts), generator=g)
    if mode == "hotspot":
        scores[:, 0] += 2.0
        scores[:, num_experts // 2] += 1.0
    idx = torch.topk(scores, topk, dim=1).indices
    if mode == "normal":
        idx = torch.sort(idx, dim=1).values
    if mode in ("invalid", "empty"):
        drop = torch.rand((tokens, topk), generator=g) < 0.3
        idx = torch.where(drop, torch.full_like(idx, -1), idx)
    if mode == "empty":
        idx[:: 3] = -1
    return idx.to(torch.int64)


from deepep_b200.utils.routing import group_limited_routes  # noqa: E402,F401  (shared with the benchmarks)


def make_weights(tokens: int, topk: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed + 77)
    return torch.softmax(torch.randn((tokens, topk), generator=g), dim=1).float()


def bits_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    return torch.equal(a.view(torch.uint8), b.view(torch.uint8))
