"""V1 expand / aggregate kernels against the CPU restatement (bit-exact: copies, and fp32 sums in slot order)."""
import pytest
import torch

from deepep_b200.ops import expand as X

pytestmark = pytest.mark.gpu


def _case(R, K, L, H, seed, align):
    g = torch.Generator().manual_seed(seed)
    scores = torch.rand((R, L), generator=g)
    idx = scores.topk(K, dim=1).indices
    idx[torch.rand((R, K), generator=g) < 0.3] = -1
    counts = [int((idx == e).sum()) for e in range(L)]
    caps = [-(-c // align) * align for c in counts]
    x = torch.randn((R, H), generator=g).to(torch.bfloat16)
    w = torch.rand((R, K), generator=g)
    return x, idx, w, caps


@pytest.mark.parametrize("R,K,L,H,align", [(1, 1, 1, 64, 1), (70, 4, 6, 256, 8), (1000, 8, 32, 1024, 128), (513, 3, 200, 128, 1)])
def test_expand_and_aggregate_match_restatement(R, K, L, H, align):
    x, idx, w, caps = _case(R, K, L, H, R + K, align)
    ex_c, ew_c, h_c = X.expand(x, idx, w, caps, align)
    dev = torch.device("cuda")
    ex, ew, h = X.expand(x.to(dev), idx.to(dev), w.to(dev), caps, align)
    assert torch.equal(h.recv_to_expanded_idx.cpu(), h_c.recv_to_expanded_idx)
    assert torch.equal(h.actual_expert_counts.cpu(), h_c.actual_expert_counts) and torch.equal(h.expert_offsets.cpu(), h_c.expert_offsets)
    assert torch.equal(ex.cpu(), ex_c) and torch.equal(ew.cpu(), ew_c)
    ex2, _, h2 = X.expand(x.to(dev) * 2, handle=h)                      # cached: mapping reused
    assert h2 is h and torch.equal(ex2.cpu(), ex_c * 2)
    y = (torch.randn(ex_c.shape, generator=torch.Generator().manual_seed(1))).to(torch.bfloat16)
    rw = torch.rand((ex_c.shape[0],), generator=torch.Generator().manual_seed(2))
    for weights in (None, rw):
        a_c, v_c = X.aggregate(y, h_c, weights, rw)
        a, v = X.aggregate(y.to(dev), h, None if weights is None else weights.to(dev), rw.to(dev))
        assert torch.equal(v.cpu(), v_c)
        assert torch.equal(a.cpu(), a_c), (a.cpu().float() - a_c.float()).abs().max()


def test_fp8_rows_with_scales_and_fp16_aggregate():
    x, idx, w, caps = _case(300, 4, 8, 512, 5, 16)
    dev = torch.device("cuda")
    q, sf = x.to(torch.float8_e4m3fn), torch.rand((300, 4))
    (e_c, s_c), _, h_c = X.expand((q, sf), idx, None, caps, 16)
    (e, s), _, h = X.expand((q.to(dev), sf.to(dev)), idx.to(dev), None, caps, 16)
    assert torch.equal(e.cpu().view(torch.uint8), e_c.view(torch.uint8)) and torch.equal(s.cpu(), s_c)
    y = torch.randn((sum(caps), 512)).to(torch.float16)
    a_c, _ = X.aggregate(y, h_c)
    a, _ = X.aggregate(y.to(dev), h)
    assert torch.equal(a.cpu(), a_c)


def test_capacity_overflow_is_reported():
    x, idx, w, caps = _case(64, 2, 4, 64, 7, 1)
    dev = torch.device("cuda")
    small = [max(c - 1, 0) for c in caps]
    with pytest.raises(ValueError, match="capacity"):
        X.expand(x.to(dev), idx.to(dev), None, small, 1)
