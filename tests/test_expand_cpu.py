"""V1 expand / aggregate on the CPU restatement: ordering, capacities, cached handles, validation."""
import pytest
import torch

import deepep_b200 as deep_ep
from deepep_b200.ops import expand as X


def _case(R=37, K=4, L=5, H=64, seed=0, align=4):
    g = torch.Generator().manual_seed(seed)
    idx = torch.full((R, K), -1, dtype=torch.int64)
    for r in range(R):
        n = int(torch.randint(0, K + 1, (1,), generator=g))
        idx[r, :n] = torch.randperm(L, generator=g)[:n]
    counts = [int((idx == e).sum()) for e in range(L)]
    caps = [-(-c // align) * align for c in counts]
    x = torch.randn((R, H), generator=g).to(torch.bfloat16)
    w = torch.rand((R, K), generator=g)
    return x, idx, w, counts, caps


def test_mapping_order_and_padding():
    x, idx, w, counts, caps = _case()
    ex, ew, h = X.expand(x, idx, w, caps, 4)
    assert h.actual_expert_counts.tolist() == counts and h.num_expanded_tokens == sum(caps)
    off = h.expert_offsets.tolist()
    for e in range(len(caps)):
        rows = [(r, k) for r in range(idx.shape[0]) for k in range(idx.shape[1]) if idx[r, k] == e]    # (row, slot) order
        for j, (r, k) in enumerate(rows):
            assert h.recv_to_expanded_idx[r, k] == off[e] + j
            assert torch.equal(ex[off[e] + j], x[r]) and ew[off[e] + j] == w[r, k]
        assert not ex[off[e] + counts[e]:off[e + 1]].any() and not ew[off[e] + counts[e]:off[e + 1]].any()
    assert (h.recv_to_expanded_idx[idx < 0] == -1).all()


def test_cached_expand_and_aggregate_roundtrip():
    x, idx, w, counts, caps = _case(seed=1)
    ex, ew, h = X.expand(x, idx, w, caps, 4)
    ex2, ew2, h2 = X.expand(x * 2, topk_weights=w, handle=h)
    assert h2 is h and torch.equal(ex2, ex * 2) and torch.equal(ew2, ew)
    agg, vals = X.aggregate(ex, h, expanded_values=ew)
    n = (idx >= 0).sum(1, keepdim=True).float()
    assert torch.allclose(agg.float(), (x.float() * n).bfloat16().float(), rtol=2e-2, atol=1e-2)
    assert torch.equal(vals, torch.where(idx >= 0, w, torch.zeros(())))
    weighted, _ = X.aggregate(ex, h, topk_weights=ew)
    expect = (x.float() * torch.where(idx >= 0, w, torch.zeros(())).sum(1, keepdim=True))
    assert torch.allclose(weighted.float(), expect, rtol=3e-2, atol=2e-2)


def test_scales_travel_with_rows():
    x, idx, w, counts, caps = _case(seed=2, H=128)
    q = x.to(torch.float8_e4m3fn)
    sf = torch.rand((x.shape[0], 1))
    (ex, esf), _, h = X.expand((q, sf), idx, None, caps, 4)
    rows, slots = (idx >= 0).nonzero(as_tuple=True)
    d = h.recv_to_expanded_idx[rows, slots].long()
    assert torch.equal(ex.view(torch.uint8)[d], q.view(torch.uint8)[rows]) and torch.equal(esf[d], sf[rows])


def test_validation():
    x, idx, w, counts, caps = _case(seed=3)
    with pytest.raises(ValueError, match="aligned"):
        X.expand(x, idx, w, [c + 1 for c in caps], 4)
    with pytest.raises(ValueError, match="capacity"):
        X.expand(x, idx, w, [0] * len(caps), 4)
    with pytest.raises(ValueError, match="recv_topk_idx is required"):
        X.expand(x, None, w, caps, 4)
    _, _, h = X.expand(x, idx, w, caps, 4)
    with pytest.raises(ValueError, match="recv_topk_idx=None"):
        X.expand(x, idx, w, handle=h)
    with pytest.raises(ValueError, match="num_recv_tokens"):
        X.expand(x[:-1], handle=h)
    with pytest.raises(TypeError):
        X.aggregate(x, object())
    with pytest.raises(ValueError, match="num_expanded_tokens"):
        X.aggregate(x, h)


def test_every_argument_rejection():
    x, idx, w, counts, caps = _case(seed=5)
    _, _, h = X.expand(x, idx, w, caps, 4)
    for call, kind, message in (
            (lambda: X.expand(x, idx, w, caps, 4.0), TypeError, "integer"),
            (lambda: X.expand(x, idx, w, caps, 0), ValueError, "positive"),
            (lambda: X.expand(x, idx, w, [], 4), TypeError, "non-empty"),
            (lambda: X.expand(x, idx, w, [float(c) for c in caps], 4), TypeError, "integers"),
            (lambda: X.expand(x, idx, w, [-4] + caps[1:], 4), ValueError, "nonnegative"),
            (lambda: X.expand(x.t().contiguous().t(), idx, w, caps, 4), ValueError, "contiguous"),
            (lambda: X.expand((x, torch.ones((x.shape[0] + 1, 1))), idx, w, caps, 4), ValueError, "scales"),
            (lambda: X.expand(x, idx, w, None, 4), ValueError, "num_tokens_per_expert is required"),
            (lambda: X.expand(x, idx.to(torch.int32), w, caps, 4), ValueError, "int64"),
            (lambda: X.expand(x, idx, w.double(), caps, 4), ValueError, "fp32"),
            (lambda: X.expand(x, handle=object()), TypeError, "ExpandHandle"),
            (lambda: X.expand(x, num_tokens_per_expert=caps, handle=h), ValueError, "num_tokens_per_expert=None"),
            (lambda: X.expand(x, expert_alignment=8, handle=h), ValueError, "match the handle")):
        with pytest.raises(kind, match=message):
            call()
    assert X.expand(x, expert_alignment=4, handle=h)[2] is h              # the handle's own alignment is accepted


def test_buffer_methods_return_events():
    x, idx, w, counts, caps = _case(seed=4)
    buf = deep_ep.Buffer(None)
    ex, ew, h, ev = buf.expand(x, idx, w, caps, 4)
    agg, vals, ev2 = buf.aggregate(ex, h, expanded_values=ew)
    assert isinstance(ev, deep_ep.EventOverlap) and isinstance(ev2, deep_ep.EventOverlap) and agg.shape == x.shape
