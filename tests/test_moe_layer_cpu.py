"""EP MoE layer forward + backward by handle reversal (Gloo, world 2) against single-process autograd."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import make_weights


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


T, H, I, E, K = 48, 64, 32, 8, 3


def _inputs(rank):
    g = torch.Generator().manual_seed(rank)
    x = torch.randn((T, H), generator=g).bfloat16()
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int64)
    return x, idx, make_weights(T, K, rank)


def _dense_reference(xs, idxs, ws, w1, w2, grads):
    """All tokens of all ranks through all experts in one process; returns per-rank (y, dx, dw) and weight grads."""
    w1 = w1.float().requires_grad_()
    w2 = w2.float().requires_grad_()
    outs = []
    for x, idx, w, g in zip(xs, idxs, ws, grads):
        xr, wr = x.float().requires_grad_(), w.clone().requires_grad_()
        y = torch.zeros((T, H))
        for k in range(K):
            for e in range(E):
                tok = (idx[:, k] == e).nonzero(as_tuple=True)[0]
                if tok.numel():
                    gate, up = (xr[tok] @ w1[e].t()).chunk(2, dim=-1)
                    y = y.index_add(0, tok, wr[tok, k].unsqueeze(1) * ((torch.nn.functional.silu(gate) * up) @ w2[e].t()))
        y.backward(g.float())
        outs.append((y.detach(), xr.grad, wr.grad))
    return outs, w1.grad, w2.grad


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=__import__("datetime").timedelta(seconds=120))
    from deepep_b200 import ElasticBuffer
    from deepep_b200.models.moe_layer import ExpertParallelMoE

    torch.manual_seed(0)
    full_w1 = (torch.randn(E, 2 * I, H) * 0.1).bfloat16()
    full_w2 = (torch.randn(E, H, I) * 0.1).bfloat16()
    buf = ElasticBuffer(dist.group.WORLD, num_max_tokens_per_rank=512, hidden=H, num_topk=K, explicitly_destroy=True)
    layer = ExpertParallelMoE(buf, E, H, I)
    L = E // world
    with torch.no_grad():
        layer.w1.copy_(full_w1[rank * L:(rank + 1) * L])
        layer.w2.copy_(full_w2[rank * L:(rank + 1) * L])
    ins = [_inputs(r) for r in range(world)]
    grads = [torch.randn((T, H), generator=torch.Generator().manual_seed(50 + r)).bfloat16() for r in range(world)]
    x, idx, w = ins[rank]
    x = x.clone().requires_grad_()
    w = w.clone().requires_grad_()
    y = layer(x, idx, w)
    y.backward(grads[rank])
    ref, g1, g2 = _dense_reference([i[0] for i in ins], [i[1] for i in ins], [i[2] for i in ins], full_w1, full_w2, grads)
    ry, rdx, rdw = ref[rank]
    ok = torch.allclose(y.float(), ry, rtol=0.05, atol=0.05)
    ok = ok and torch.allclose(x.grad.float(), rdx, rtol=0.05, atol=0.05)
    ok = ok and torch.allclose(w.grad, rdw, rtol=0.05, atol=0.08)
    ok = ok and torch.allclose(layer.w1.grad.float(), g1[rank * L:(rank + 1) * L], rtol=0.05, atol=0.08)
    ok = ok and torch.allclose(layer.w2.grad.float(), g2[rank * L:(rank + 1) * L], rtol=0.05, atol=0.08)
    buf.destroy()
    results[rank] = bool(ok)
    dist.destroy_process_group()


def test_moe_layer_forward_backward():
    world, port = 2, _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: True, 1: True}
