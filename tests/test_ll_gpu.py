"""Low-latency dispatch/combine kernels: virtual ranks on one GPU against the oracle, and CUDA-graph replay."""
import pytest
import torch

from deepep_b200.oracle import reference as R
from deepep_b200.utils.math import per_token_cast_to_fp8
from helpers import bits_equal, make_routes, make_weights

pytestmark = pytest.mark.gpu


def _case(world, tokens, H, E, K, mode, routes="random", repeats=2):
    from deepep_b200.parallel.virtual import VirtualWorld
    from deepep_b200.ops import load_native

    C = load_native()
    dev = torch.device("cuda")
    M = max(max(tokens), 1)
    with VirtualWorld(world, M, H, K, timeout=10.0, ll_bytes=C.ll_region_bytes(world, M, K, H)) as vw:
        eng = vw.engine
        for rep in range(repeats):
            xs = [torch.randn((t, H), generator=torch.Generator().manual_seed(rep * 100 + r)).bfloat16() for r, t in enumerate(tokens)]
            idx = [make_routes(routes, t, E, K, world, rep * 10 + r) for r, t in enumerate(tokens)]
            ws = [make_weights(t, K, rep + r) for r, t in enumerate(tokens)]
            if mode == 1:
                q = [per_token_cast_to_fp8(x) for x in xs]
                dx, rx_in = [(a.to(dev), b.to(dev)) for a, b in q], q
            else:
                dx, rx_in = [x.to(dev) for x in xs], xs
            res = eng.ll_dispatch(dx, [i.to(dev) for i in idx], [w.to(dev) for w in ws], E, mode)
            ref, lays = R.dispatch(rx_in, idx, ws, E, do_expand=True, quantize_fp8=(mode == 2))
            for r in range(world):
                plan, rx, rsf = res[r]
                assert plan.num_rows == lays[r].num_rows
                assert plan.expert_counts_list == lays[r].expert_counts.tolist()
                if mode == 0:
                    assert bits_equal(rx, ref[r][0])
                else:
                    assert bits_equal(rx, ref[r][0][0]) and bits_equal(rsf, ref[r][0][1])
                assert torch.equal(plan.recv_w[:plan.num_rows].cpu(), ref[r][2])
            eouts = [torch.randn((lays[r].num_rows, H), generator=torch.Generator().manual_seed(7 + r)).bfloat16() for r in range(world)]
            outs = eng.ll_combine([e.to(dev) for e in eouts], [res[r][0] for r in range(world)])
            cref = R.low_latency_combine(eouts, lays, ws, tokens)
            torch.cuda.synchronize()
            eng.check_status()
            for r in range(world):
                assert bits_equal(outs[r], cref[r]), f"rank {r} combined output differs"


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ll_bf16(world):
    _case(world, [100 + 7 * r for r in range(world)], 1024, 16 * world, 4, 0, repeats=3)


def test_ll_invalid_and_empty():
    _case(4, [128, 0, 5, 256], 512, 32, 8, 0, routes="empty")


def test_ll_fp8():
    _case(2, [128, 77], 2048, 32, 8, 1)
    _case(2, [128, 77], 2048, 32, 8, 2)


def test_ll_decode_shape():
    _case(8, [128] * 8, 7168, 384, 8, 2, repeats=1)


def test_ll_graph_replay_public_api():
    """dispatch + combine through ElasticBuffer inside one captured CUDA graph, replayed with new inputs."""
    from deepep_b200 import ElasticBuffer

    dev = torch.device("cuda")
    T, H, E, K = 64, 1024, 16, 4
    buf = ElasticBuffer(None, num_max_tokens_per_rank=128, hidden=H, num_topk=K, explicitly_destroy=True)
    x = torch.zeros((T, H), dtype=torch.bfloat16, device=dev)
    idx = torch.zeros((T, K), dtype=torch.int64, device=dev)
    w = torch.zeros((T, K), dtype=torch.float32, device=dev)

    def fill(seed):
        x.copy_(torch.randn((T, H), generator=torch.Generator().manual_seed(seed)).bfloat16())
        idx.copy_(make_routes("random", T, E, K, 1, seed))
        w.copy_(make_weights(T, K, seed))

    def step():
        rx, _, rw, handle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_cpu_sync=False)
        assert handle.is_low_latency
        out, _, _ = buf.combine(rx, handle)
        return out

    fill(0)
    for _ in range(2):
        step()           # warm up outside the graph
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = step()
    for seed in (1, 2, 3):
        fill(seed)
        graph.replay()
        torch.cuda.synchronize()
        ok = make_routes("random", T, E, K, 1, seed) >= 0
        expect = x.float().cpu() * (make_weights(T, K, seed) * ok).sum(1, keepdim=True)
        assert torch.allclose(out.float().cpu(), expect, rtol=0.02, atol=0.05)
    buf.destroy()


def test_ll_empty_batch_takes_the_same_path():
    """The path is chosen from the buffer and the options, never from a rank's own token count: an empty batch on a
    decode buffer runs the low-latency kernels too (with peers, a rank that chose differently would never be answered)."""
    from deepep_b200 import ElasticBuffer

    dev = torch.device("cuda")
    H, E, K = 512, 16, 4
    buf = ElasticBuffer(None, num_max_tokens_per_rank=64, hidden=H, num_topk=K, explicitly_destroy=True)
    x = torch.zeros((0, H), dtype=torch.bfloat16, device=dev)
    idx = torch.zeros((0, K), dtype=torch.int64, device=dev)
    w = torch.zeros((0, K), dtype=torch.float32, device=dev)
    rx, _, rw, handle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E)
    assert handle.is_low_latency and rx.shape == (0, H) and handle.num_recv_tokens_per_expert_list == [0] * E
    out, _, _ = buf.combine(rx, handle)
    torch.cuda.synchronize()
    assert out.shape == (0, H)
    buf.destroy()
