"""ElasticBuffer over Gloo on CPU, world size 2: dispatch -> weighted identity experts -> combine, and its backward."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import make_weights


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _routes(tokens, experts, topk, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn((tokens, experts), generator=g)
    probs = torch.softmax(logits, dim=1)
    w, idx = torch.topk(probs, topk, dim=1)
    return idx.to(torch.int64), (w / w.sum(dim=1, keepdim=True)).float()


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=__import__("datetime").timedelta(seconds=120))
    import deepep_b200 as deep_ep

    T, H, E, K = 128, 512, 16, 4
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(rank)).bfloat16()
    idx, w = _routes(T, E, K, 100 + rank)
    buf = deep_ep.ElasticBuffer(dist.group.WORLD, num_max_tokens_per_rank=T, hidden=H, num_topk=K, explicitly_destroy=True,
                                debug_collectives=True)
    recv_x, recv_idx, recv_w, handle, event = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True)
    assert recv_idx is None and recv_w.shape == (recv_x.shape[0],)
    assert sum(handle.num_recv_tokens_per_expert_list) == recv_x.shape[0]
    expert_out = (recv_x.float() * recv_w.unsqueeze(1)).bfloat16()
    combined, cw, _ = buf.combine(expert_out, handle, topk_weights=recv_w)
    expect = x.float() * w.sum(dim=1, keepdim=True)
    ok = torch.allclose(combined.float(), expect, rtol=0.01, atol=0.03125) and torch.equal(cw, w)
    # backward by handle reversal: d(combine)/dx = dispatch(grad, handle); d(dispatch)/dx = combine(grad_recv, handle)
    grad_out = torch.randn((T, H), generator=torch.Generator().manual_seed(7 + rank)).bfloat16()
    grad_rows, _, _, _, _ = buf.dispatch(grad_out, handle=handle)
    assert grad_rows.shape == recv_x.shape
    grad_x, grad_w, _ = buf.combine((grad_rows.float() * recv_w.unsqueeze(1)).bfloat16(), handle,
                                    topk_weights=(grad_rows.float() * recv_x.float()).sum(dim=1))
    # autograd reference of y = sum_k w_k x
    xr, wr = x.float().requires_grad_(), w.clone().requires_grad_()
    (xr * wr.sum(dim=1, keepdim=True)).backward(grad_out.float())
    ok = ok and torch.allclose(grad_x.float(), xr.grad, rtol=0.02, atol=0.06)
    ok = ok and torch.allclose(grad_w, wr.grad, rtol=0.02, atol=0.5)
    # rank layout (do_expand=False)
    rx2, ridx2, rw2, h2, _ = buf.dispatch(x, topk_idx=idx, num_experts=E, do_expand=False)
    assert ridx2.shape == (rx2.shape[0], K) and rw2 is None
    c2, _, _ = buf.combine(rx2, h2)
    dests = torch.stack([(torch.div(idx, E // world, rounding_mode="floor") == d).any(dim=1) for d in range(world)], 1).sum(1)
    ok = ok and torch.allclose(c2.float(), x.float() * dests.unsqueeze(1), rtol=0.01, atol=0.03125)
    buf.destroy()
    results[rank] = bool(ok)
    dist.destroy_process_group()


def test_gloo_world2_roundtrip_and_backward():
    world, port = 2, _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: True, 1: True}


def test_single_process_buffer_and_errors():
    import deepep_b200 as deep_ep

    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    buf = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=32, hidden=64, num_topk=2, explicitly_destroy=True)
    x = torch.randn(32, 64).bfloat16()
    idx = torch.randint(0, 4, (32, 2)).to(torch.int64)
    idx[:, 1] = (idx[:, 0] + 1) % 4
    w = make_weights(32, 2)
    rx, _, rw, h, ev = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=4)
    assert h.is_low_latency and ev.event is None
    out, ow, _ = buf.combine((rx.float() * 1.0).bfloat16(), h)
    assert ow is None and torch.allclose(out.float(), x.float() * w.sum(1, keepdim=True), rtol=0.02, atol=0.05)
    with pytest.raises(ValueError):
        buf.dispatch(x, topk_idx=idx, num_experts=4, handle=h)
    with pytest.raises(ValueError):
        buf.dispatch(x[:, :32], topk_idx=idx, num_experts=4)
    with pytest.raises(NotImplementedError):
        buf.pp_send()
    h.topk_idx.add_(0)
    with pytest.raises(RuntimeError):
        buf.combine(rx, h)
    buf.destroy()
    buf.destroy()
    with pytest.raises(RuntimeError):
        buf.dispatch(x, topk_idx=idx, num_experts=4)
