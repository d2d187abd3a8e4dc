"""Upstream V1 ``Buffer`` on the CPU engine: layout, dispatch with the six-tensor handle, combine, slot life cycle."""
import pytest
import torch

import deepep_b200 as deep_ep
from deepep_b200.resources import Handle, SlotPool, SlotState
from helpers import make_routes, make_weights


def test_slot_life_cycle_and_generations():
    pool = SlotPool(2)
    a = pool.acquire()
    assert a.state is SlotState.ACQUIRED and a.generation == 1
    a.move(SlotState.DISPATCH_IN_FLIGHT)
    with pytest.raises(RuntimeError, match="illegal transition"):
        a.move(SlotState.RELEASABLE)
    a.move(SlotState.DISPATCH_READY)
    b = pool.acquire()
    b.move(SlotState.DISPATCH_IN_FLIGHT)
    c = pool.acquire()                       # both slots taken: the finished dispatch (a) gives way, b is in flight
    assert c is a and a.generation == 2
    with pytest.raises(RuntimeError, match="in flight"):
        pool.acquire()
    pool.release(b)
    assert b.state is SlotState.FREE


def test_layout_dispatch_combine_and_stale_handles():
    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    T, H, E, K = 70, 64, 8, 3
    x = torch.randn(T, H).bfloat16()
    idx, w = make_routes("invalid", T, E, K, 1, 3), make_weights(T, K, 1)
    buf = deep_ep.Buffer(None, num_max_tokens_per_rank=128, hidden=H, num_topk=K)
    per_rank, per_rdma, per_expert, in_rank, ev = buf.get_dispatch_layout(idx, E)
    assert per_rdma is None and per_rank.tolist() == [int((idx >= 0).any(1).sum())]
    assert per_expert.tolist() == torch.bincount(idx[idx >= 0], minlength=E).tolist() and in_rank.shape == (T, 1)
    rx, ridx, rw, counts, handle, ev = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_rank=per_rank,
                                                    is_token_in_rank=in_rank, num_tokens_per_expert=per_expert, expert_alignment=4)
    assert isinstance(handle, Handle) and len(handle) == 6
    rank_prefix, chan_prefix, recv_chan_prefix, recv_src_idx, in_rank2, send_head = handle
    assert rank_prefix.tolist() == [[rx.shape[0]]] and recv_src_idx.shape == (rx.shape[0],)
    assert torch.equal(in_rank2, in_rank) and send_head.shape == (T, 1)
    assert torch.equal(rx, x[recv_src_idx.long()])                                   # rows are the tokens they name
    assert chan_prefix.tolist() == [[0, int(in_rank[:64].sum())]] and recv_chan_prefix[0, 1] == int(in_rank[:64].sum())
    assert all(c % 4 == 0 for c in counts) and sum(counts) >= int((ridx >= 0).sum())
    out, ow, _ = buf.combine(rx, handle, topk_weights=rw)
    assert torch.allclose(out.float(), x.float() * in_rank.float(), rtol=0.01, atol=0.02)
    assert handle.slot.state is SlotState.RELEASABLE
    # backward of combine through the same handle, then three more dispatches recycle the first slot
    again = buf.dispatch(out, handle=handle)[0]
    assert again.shape == rx.shape
    for _ in range(4):
        last = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_expert=per_expert)[4]
    with pytest.raises(RuntimeError, match="stale handle"):
        buf.combine(rx, handle)
    buf.release(last)
    with pytest.raises(RuntimeError, match="stale handle"):
        buf.combine(rx, last)
    with pytest.raises(ValueError, match="num_worst_tokens"):
        buf.dispatch(x, topk_idx=idx, num_tokens_per_expert=per_expert, num_worst_tokens=5)
    # fixed-size outputs: group size x num_max_tokens_per_rank rows, no per-expert list, the same rows first
    fx, fidx, fw, fcounts, fhandle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_expert=per_expert,
                                                     num_worst_tokens=128)
    assert fx.shape[0] == 128 and fcounts == [] and torch.equal(fx[:rx.shape[0]], rx) and not fx[rx.shape[0]:].any()
    assert torch.equal(fidx[:rx.shape[0]], ridx) and bool((fidx[rx.shape[0]:] == -1).all())
    fout, _, _ = buf.combine(fx, fhandle, topk_weights=fw)
    assert torch.equal(fout, out)
    with pytest.raises(TypeError, match="zero_copy"):
        buf.dispatch(x, topk_idx=idx, num_tokens_per_expert=per_expert, zero_copy=1)
    zc = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_expert=per_expert, zero_copy=True)[0]
    assert torch.equal(zc, rx)
    buf.destroy()
