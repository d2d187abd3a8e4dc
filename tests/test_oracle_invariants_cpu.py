"""Mathematical invariants of the all-rank oracle over randomly generated routing (hypothesis), plus a hand-calculated
anchor.  The kernels are checked against this oracle bit for bit, so what holds here is what the library promises."""
import torch
from hypothesis import given, settings, strategies as st

from deepep_b200.oracle import reference as R


@st.composite
def routing_cases(draw):
    world = draw(st.sampled_from([1, 2, 4]))
    local = draw(st.integers(1, 3))
    experts = world * local
    topk = draw(st.integers(1, min(4, experts)))
    hidden = draw(st.sampled_from([8, 16]))
    tokens = [draw(st.integers(0, 6)) for _ in range(world)]
    seed = draw(st.integers(0, 10_000))
    g = torch.Generator().manual_seed(seed)
    idx = []
    for t in tokens:
        rows = torch.stack([torch.randperm(experts, generator=g)[:topk] for _ in range(t)]) if t else torch.zeros((0, topk), dtype=torch.int64)
        rows = rows.to(torch.int64)
        mask = torch.rand(rows.shape, generator=g) < 0.25            # a quarter of the slots are masked
        idx.append(torch.where(mask, torch.full_like(rows, -1), rows))
    # small integers: every sum below is exact in bf16, so equalities can be checked bit for bit
    xs = [torch.randint(-3, 4, (t, hidden), generator=g).to(torch.bfloat16) for t in tokens]
    ws = [torch.rand((t, topk), generator=g) for t in tokens]
    align = draw(st.sampled_from([1, 1, 4]))
    return world, experts, topk, hidden, tokens, idx, xs, ws, align


@settings(max_examples=60, deadline=None, derandomize=True)
@given(routing_cases())
def test_expanded_layout_invariants(case):
    world, experts, topk, hidden, tokens, idx, xs, ws, align = case
    local = experts // world
    outs, lays = R.dispatch(xs, idx, ws, experts, do_expand=True, expert_alignment=align)
    valid_total = sum(int(((i >= 0) & (i < experts)).sum()) for i in idx)
    assert sum(int(l.expert_counts.sum()) for l in lays) == valid_total                 # every valid slot lands exactly once
    for r, (lay, (rx, _, rw)) in enumerate(zip(lays, outs)):
        # blocks start at multiples of the alignment and hold their expert's rows; padding rows are zero
        assert all(int(o) % align == 0 for o in lay.expert_offsets[:-1]) and lay.num_rows == rx.shape[0]
        padding = torch.ones(lay.num_rows, dtype=torch.bool)
        padding[lay.row_index] = False
        assert not rx[padding].any() and not rw[padding].any()
        # order inside the rank: (local expert, source rank, token, slot), strictly increasing
        keys = []
        for src, tok, slot, pos in zip(lay.row_source.tolist(), lay.row_token.tolist(), lay.row_slot.tolist(), lay.row_index.tolist()):
            e = int(idx[src][tok, slot])
            assert e // local == r
            keys.append((e % local, src, tok, slot))
            assert torch.equal(rx[pos], xs[src][tok]) and float(rw[pos]) == float(ws[src][tok, slot])
        assert keys == sorted(keys) and len(set(keys)) == len(keys)
    # identity experts: combine gives x times the number of valid slots (exact for these small integers)
    back = R.combine([o[0] for o in outs], lays, tokens, topk)
    for r in range(world):
        n_valid = ((idx[r] >= 0) & (idx[r] < experts)).sum(1, keepdim=True)
        assert torch.equal(back[r][0].float(), xs[r].float() * n_valid)


@settings(max_examples=40, deadline=None, derandomize=True)
@given(routing_cases())
def test_rank_layout_matches_expanded_layout(case):
    world, experts, topk, hidden, tokens, idx, xs, ws, _ = case
    local = experts // world
    outs, lays = R.dispatch(xs, idx, ws, experts, do_expand=False)
    eouts, elays = R.dispatch(xs, idx, ws, experts, do_expand=True)
    for r in range(world):
        rx, ridx, rw = outs[r]
        lay = lays[r]
        # one row per (source, token) that has an expert here, in (source, token) order
        pairs = list(zip(lay.row_source.tolist(), lay.row_token.tolist()))
        assert pairs == sorted(set(pairs))
        assert int(lay.rank_rows.sum()) == len(pairs) == rx.shape[0]
        for pos, (src, tok) in enumerate(pairs):
            here = [(k, int(e)) for k, e in enumerate(idx[src][tok].tolist()) if 0 <= e < experts and e // local == r]
            assert here and torch.equal(rx[pos], xs[src][tok])
            assert ridx[pos].tolist() == [e % local if (k, e) in here else -1 for k, e in enumerate(idx[src][tok].tolist())]
            assert rw[pos].tolist() == [float(ws[src][tok, k]) if (k, e) in here else 0.0 for k, e in enumerate(idx[src][tok].tolist())]
        # the expanded layout of the same routing holds one row per local slot of those rows
        assert int(elays[r].expert_counts.sum()) == int((ridx >= 0).sum())


def test_hand_calculated_anchor():
    """Two ranks, four experts (two per rank), top-2: rank 0 tokens 2 and 3, rank 1 token 5."""
    xs = [torch.tensor([[2.0], [3.0]]).bfloat16().repeat(1, 8), torch.tensor([[5.0]]).bfloat16().repeat(1, 8)]
    idx = [torch.tensor([[0, 1], [2, -1]]), torch.tensor([[1, 3]])]
    ws = [torch.tensor([[0.25, 0.5], [0.75, 9.0]]), torch.tensor([[0.125, 0.625]])]
    outs, lays = R.dispatch(xs, idx, ws, 4, do_expand=True)
    assert lays[0].expert_counts.tolist() == [1, 2] and lays[1].expert_counts.tolist() == [1, 1]
    assert outs[0][0][:, 0].tolist() == [2.0, 2.0, 5.0] and outs[0][2].tolist() == [0.25, 0.5, 0.125]
    assert outs[1][0][:, 0].tolist() == [3.0, 5.0] and outs[1][2].tolist() == [0.75, 0.625]
    ranked, _ = R.dispatch(xs, idx, ws, 4, do_expand=False)
    assert ranked[0][0][:, 0].tolist() == [2.0, 5.0] and ranked[0][1].tolist() == [[0, 1], [1, -1]]
    assert ranked[1][0][:, 0].tolist() == [3.0, 5.0] and ranked[1][1].tolist() == [[0, -1], [-1, 1]]
    assert ranked[1][2].tolist() == [[0.75, 0.0], [0.0, 0.625]]          # masked and remote slots carry weight zero
    weighted = [(o[0].float() * o[2].unsqueeze(1)).bfloat16() for o in outs]
    back = R.combine(weighted, lays, [2, 1], 2)
    assert back[0][0][:, 0].tolist() == [1.5, 2.25] and back[1][0][:, 0].tolist() == [3.75]


@settings(max_examples=40, deadline=None, derandomize=True)
@given(routing_cases())
def test_low_latency_combine_is_the_weighted_sum(case):
    """Identity experts and weights that are powers of two (products and sums exact): the low-latency combine returns
    ``x * sum of the weights of the valid slots``, and so does the layout-free restatement."""
    world, experts, topk, hidden, tokens, idx, xs, _, _ = case
    g = torch.Generator().manual_seed(sum(tokens) + experts)
    ws = [torch.tensor(2.0) ** torch.randint(-3, 2, (t, topk), generator=g).float() for t in tokens]
    outs, lays = R.dispatch(xs, idx, ws, experts, do_expand=True)
    back = R.low_latency_combine([o[0] for o in outs], lays, ws, tokens)
    want = R.expected_roundtrip(xs, idx, ws, experts)
    for r in range(world):
        assert torch.equal(back[r].float(), want[r])
