"""Training path on GPUs: ExpertParallelMoE forward + backward by handle reversal against a dense autograd model that
holds every expert in one process (bf16 input gradients, fp32 top-k weight gradients, expert weight gradients)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import make_weights

pytestmark = pytest.mark.gpu

T, H, I, E, K = 200, 512, 256, 16, 4


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(rank):
    g = torch.Generator().manual_seed(rank)
    x = torch.randn((T, H), generator=g).bfloat16()
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int64)
    return x, idx, make_weights(T, K, rank)


def _dense(xs, idxs, ws, w1, w2, grads, dev):
    """Every token of every rank through every expert on one GPU in fp32."""
    w1 = w1.float().to(dev).requires_grad_()
    w2 = w2.float().to(dev).requires_grad_()
    outs = []
    for x, idx, w, g in zip(xs, idxs, ws, grads):
        xr, wr, idx = x.float().to(dev).requires_grad_(), w.clone().to(dev).requires_grad_(), idx.to(dev)
        y = torch.zeros((T, H), device=dev)
        for k in range(K):
            for e in range(E):
                tok = (idx[:, k] == e).nonzero(as_tuple=True)[0]
                if tok.numel():
                    gate, up = (xr[tok] @ w1[e].t()).chunk(2, dim=-1)
                    y = y.index_add(0, tok, wr[tok, k].unsqueeze(1) * ((torch.nn.functional.silu(gate) * up) @ w2[e].t()))
        y.backward(g.float().to(dev))
        outs.append((y.detach(), xr.grad, wr.grad))
    return outs, w1.grad, w2.grad


def _run(rank, world, group, dev, grouped):
    from deepep_b200 import ElasticBuffer
    from deepep_b200.models.moe_layer import ExpertParallelMoE

    torch.manual_seed(0)
    full_w1 = (torch.randn(E, 2 * I, H) * 0.05).bfloat16()
    full_w2 = (torch.randn(E, H, I) * 0.05).bfloat16()
    buf = ElasticBuffer(group, num_max_tokens_per_rank=512, hidden=H, num_topk=K, explicitly_destroy=True)
    layer = ExpertParallelMoE(buf, E, H, I, device=dev)
    layer.use_grouped_mm = grouped
    L = E // world
    with torch.no_grad():
        layer.w1.copy_(full_w1[rank * L:(rank + 1) * L])
        layer.w2.copy_(full_w2[rank * L:(rank + 1) * L])
    ins = [_inputs(r) for r in range(world)]
    grads = [torch.randn((T, H), generator=torch.Generator().manual_seed(50 + r)).bfloat16() for r in range(world)]
    x, idx, w = ins[rank]
    x = x.to(dev).requires_grad_()
    w = w.to(dev).requires_grad_()
    y = layer(x, idx.to(dev), w)
    y.backward(grads[rank].to(dev))
    torch.cuda.synchronize()
    ref, g1, g2 = _dense([i[0] for i in ins], [i[1] for i in ins], [i[2] for i in ins], full_w1, full_w2, grads, dev)
    ry, rdx, rdw = ref[rank]
    def close(a, b):   # bf16 rounding of the products scales with the tensor, not with each element
        return bool((a.float() - b).abs().max() <= 0.02 * b.abs().max())

    checks = dict(y=close(y, ry), dx=close(x.grad, rdx), dw=close(w.grad, rdw),
                  dw1=close(layer.w1.grad, g1[rank * L:(rank + 1) * L]), dw2=close(layer.w2.grad, g2[rank * L:(rank + 1) * L]),
                  dtypes=x.grad.dtype == torch.bfloat16 and w.grad.dtype == torch.float32)
    buf.destroy()
    return checks


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    results[rank] = _run(rank, world, dist.group.WORLD, dev, False)
    dist.destroy_process_group()


@pytest.mark.parametrize("grouped", [False, True])
def test_one_gpu_matches_dense_autograd(grouped):
    from deepep_b200.utils.grouped_mm import grouped_mm_usable

    if grouped and not grouped_mm_usable():
        pytest.skip("this PyTorch build has no usable grouped GEMM for the device")
    checks = _run(0, 1, None, torch.device("cuda"), grouped)
    assert all(checks.values()), checks


@pytest.mark.parametrize("world", [2, 4, 8])
def test_real_ranks_match_dense_autograd(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        res = dict(results)
    assert all(all(res[r].values()) for r in range(world)), res
