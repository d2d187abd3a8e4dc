"""The library baseline (all-to-all-v formulation) agrees with the oracle on one process (world size 1, CPU tensors)."""
import torch

from baseline.nccl_moe import ExpertWeights, NcclExpertParallel, moe_forward
from helpers import make_routes, make_weights


def test_single_process_roundtrip():
    T, H, E, K = 64, 32, 8, 3
    x = torch.randn(T, H).bfloat16()
    idx, w = make_routes("invalid", T, E, K, 1, 0), make_weights(T, K, 0)
    ep = NcclExpertParallel(None, E)
    plan = ep.plan(idx, w)
    rows = ep.dispatch(x, plan)
    out = ep.combine(rows, plan)
    expect = x.float() * (w * (idx >= 0)).sum(1, keepdim=True)
    assert torch.allclose(out.float(), expect, rtol=0.02, atol=0.05)


def test_moe_forward_matches_dense_loop():
    T, H, I, E, K = 32, 16, 8, 4, 2
    x = torch.randn(T, H)
    idx, w = make_routes("random", T, E, K, 1, 1), make_weights(T, K, 1)
    w1, w2 = torch.randn(E, 2 * I, H) * 0.2, torch.randn(E, H, I) * 0.2
    ep = NcclExpertParallel(None, E)
    y = moe_forward(ep, x.bfloat16(), ep.plan(idx, w), ExpertWeights(w1.bfloat16(), w2.bfloat16()))
    ref = torch.zeros(T, H)
    for t in range(T):
        for k in range(K):
            e = int(idx[t, k])
            g, u = (x[t] @ w1[e].t()).chunk(2)
            ref[t] += w[t, k] * ((torch.nn.functional.silu(g) * u) @ w2[e].t())
    assert torch.allclose(y.float(), ref, rtol=0.05, atol=0.1)
