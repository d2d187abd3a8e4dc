"""Properties of the public ``ElasticBuffer`` API over generated shapes and routings (hypothesis, one process, CPU
engine): whatever the layout, the alignment or the path, a round trip through identity experts returns ``x`` times
the number of rows the token was sent as, the handle's counts describe the rows, cached dispatches repeat the
fresh one, and the weights channel returns what was sent.  Small integers keep every sum exact in bf16."""
import pytest
import torch
from hypothesis import given, settings, strategies as st

import deepep_b200 as deep_ep


@st.composite
def calls(draw):
    experts = draw(st.sampled_from([1, 2, 4, 6, 9]))
    topk = draw(st.integers(1, min(4, experts)))
    hidden = draw(st.sampled_from([8, 64, 128]))
    cap = draw(st.sampled_from([16, 300]))                         # 16: a decode buffer (low latency possible); 300: not
    tokens = draw(st.integers(0, 12))
    seed = draw(st.integers(0, 10_000))
    g = torch.Generator().manual_seed(seed)
    idx = torch.stack([torch.randperm(experts, generator=g)[:topk] for _ in range(tokens)]).to(torch.int64) if tokens \
        else torch.zeros((0, topk), dtype=torch.int64)
    idx = torch.where(torch.rand(idx.shape, generator=g) < 0.25, torch.full_like(idx, -1), idx)
    x = torch.randint(-3, 4, (tokens, hidden), generator=g).to(torch.bfloat16)
    w = torch.randint(1, 5, (tokens, topk), generator=g).float()
    return experts, topk, hidden, cap, idx, x, w, draw(st.booleans()), draw(st.sampled_from([1, 1, 8])), draw(st.booleans())


@settings(max_examples=80, deadline=None, derandomize=True)
@given(calls())
def test_round_trip_properties(case):
    experts, topk, hidden, cap, idx, x, w, expand, align, with_weights = case
    if not expand:
        align = 1
    tokens = x.shape[0]
    valid = (idx >= 0).sum(1, keepdim=True).float()
    buf = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=cap, hidden=hidden, num_topk=topk, explicitly_destroy=True, device="cpu")
    try:
        rx, ridx, rw, handle, event = buf.dispatch(x, topk_idx=idx, topk_weights=w if with_weights else None, num_experts=experts,
                                                   do_expand=expand, expert_alignment=align if align > 1 else None)
        assert event.event is None and handle.num_experts == experts
        counts = handle.num_recv_tokens_per_expert_list
        assert counts == torch.bincount(idx[idx >= 0], minlength=experts).tolist()           # one rank owns every expert
        low_latency = handle.is_low_latency
        assert low_latency == (cap <= 256 and with_weights and not expand)
        if expand or low_latency:
            aligned = [-(-c // align) * align for c in counts]
            assert rx.shape[0] == sum(aligned) and ridx is None
            assert handle.psum_num_recv_tokens_per_expert.tolist() == torch.tensor(aligned).cumsum(0).tolist()
            assert (rw is None) == (not with_weights) and (rw is None or rw.shape == (rx.shape[0],))
        else:
            assert rx.shape[0] == int((valid > 0).sum()) and tuple(ridx.shape) == (rx.shape[0], topk)
            assert torch.equal(ridx, idx[(idx >= 0).any(1)])                                 # local ids = global ids on one rank
            assert (rw is None) == (not with_weights)
        again = buf.dispatch(x * 2, handle=handle)[0]
        assert torch.equal(again.float(), rx.float() * 2)
        if low_latency:
            out, out_w, _ = buf.combine(rx, handle)                                          # applies the saved weights
            want = x.float() * torch.where(idx >= 0, w, torch.zeros_like(w)).sum(1, keepdim=True)
            assert out_w is None and torch.equal(out.float(), want.bfloat16().float())
        else:
            out, out_w, _ = buf.combine(rx, handle, topk_weights=rw)
            # expanded: one row per valid slot; rank layout: one row per destination rank (here at most one)
            copies = valid if expand else (valid > 0).float()
            assert torch.equal(out.float(), x.float() * copies) and out.shape == (tokens, hidden)
            if with_weights:
                assert torch.equal(out_w, torch.where(idx >= 0, w, torch.zeros_like(w)))
            else:
                assert out_w is None
    finally:
        buf.destroy()


@settings(max_examples=40, deadline=None, derandomize=True)
@given(calls())
def test_outputs_without_a_read_back_of_the_counts(case):
    """``do_cpu_sync=False``: nothing is read back, so outputs have the worst-case number of rows; the first rows are those
    of the synchronous call, the rest carries no data, the handle has no per-expert list, and combine takes the rows as
    they came and returns the same result."""
    experts, topk, hidden, cap, idx, x, w, expand, align, with_weights = case
    if not expand:
        align = 1
    buf = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=cap, hidden=hidden, num_topk=topk, explicitly_destroy=True, device="cpu")
    try:
        kwargs = dict(topk_idx=idx, topk_weights=w if with_weights else None, num_experts=experts, do_expand=expand,
                      expert_alignment=align if align > 1 else None)
        rx, ridx, rw, handle, _ = buf.dispatch(x, **kwargs)
        fx, fidx, fw, fixed, _ = buf.dispatch(x, do_cpu_sync=False, **kwargs)
        expanded = expand or fixed.is_low_latency
        worst = cap * (min(topk, experts) if expanded else 1) + (experts * (align - 1) if align > 1 else 0)
        exact = rx.shape[0]
        assert fx.shape[0] == worst >= exact and fixed.num_recv_tokens_per_expert_list is None
        assert torch.equal(fx[:exact], rx) and not fx[exact:].any()
        assert (fw is None) == (rw is None) and (fw is None or (fw.shape[0] == worst and torch.equal(fw[:exact], rw)))
        assert (fidx is None) == (ridx is None) and (fidx is None or torch.equal(fidx[:exact], ridx))
        out, out_w, _ = buf.combine(rx, handle, topk_weights=None if handle.is_low_latency else rw)
        out2, out_w2, _ = buf.combine(fx, fixed, topk_weights=None if fixed.is_low_latency else fw)
        assert torch.equal(out, out2) and (out_w is None) == (out_w2 is None) and (out_w is None or torch.equal(out_w, out_w2))
        with pytest.raises(ValueError, match="rows"):
            buf.combine(fx[:exact] if exact != worst else fx[:-1], fixed)
    finally:
        buf.destroy()
