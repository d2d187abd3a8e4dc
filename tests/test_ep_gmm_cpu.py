"""ep_gmm_fused public API on the CPU engine (Gloo ranks) and the restatement's own consistency."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deepep_b200.ops import ep_gmm_fused as G


def test_restatements_are_inverse_layouts():
    world, E, K = 2, 4, 64
    counts = [[3, 0, 2, 5], [1, 4, 0, 2]]
    xs = [torch.arange(sum(c) * K, dtype=torch.float32).view(-1, K).to(torch.bfloat16) + 1000 * s for s, c in enumerate(counts)]
    eye = torch.eye(K, dtype=torch.bfloat16).expand(E // world, K, K).contiguous()
    outs, gathered = G.reference_alltoallv_gmm(xs, [eye] * world, counts, E)
    for o, g in zip(outs, gathered):
        assert torch.equal(o, g)
    back = G.reference_gmm_alltoallv(gathered, [eye] * world, counts, E)
    for b, x in zip(back, xs):
        assert torch.equal(b, x)


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        E, K, N = 4, 64, 128
        counts = [[3, 0, 2, 5], [1, 4, 0, 2]]
        L = E // world
        gen = torch.Generator().manual_seed(11)
        xs = [torch.randn((sum(c), K), generator=gen).to(torch.bfloat16) for c in counts]
        ws = [torch.randn((L, K, N), generator=gen).to(torch.bfloat16) / 8 for _ in range(world)]
        cfg = G.init_group(dist.group.WORLD, max_rows=64, max_k=K, max_n=N, device="cpu")
        assert cfg.backend == "cpu" and cfg.world_size == world and G.get_udma_config() == cfg
        glob = [counts[s][rank * L + l] for s in range(world) for l in range(L)]
        out, gathered = G.alltoallv_gmm(xs[rank], ws[rank], counts[rank], glob, ep_size=world, expert_num=E, output_all_to_allv=True)
        ref_out, ref_g = G.reference_alltoallv_gmm(xs, ws, counts, E)
        assert torch.equal(out, ref_out[rank]) and torch.equal(gathered, ref_g[rank])
        ws2 = [torch.randn((L, K, K), generator=gen).to(torch.bfloat16) / 8 for _ in range(world)]
        back = G.gmm_alltoallv(gathered, ws2[rank], torch.tensor(counts[rank]), torch.tensor(glob), ep_size=world, expert_num=E)
        assert torch.equal(back, G.reference_gmm_alltoallv(ref_g, ws2, counts, E)[rank])
        with pytest.raises(ValueError):
            G.alltoallv_gmm(xs[rank][:1], ws[rank], counts[rank], glob, ep_size=world, expert_num=E)
        with pytest.raises(ValueError):
            G.gmm_alltoallv(gathered, ws2[rank], counts[rank], glob, ep_size=world + 1, expert_num=E)
        G.destroy_group()
        with pytest.raises(RuntimeError):
            G.get_config()
        results[rank] = "ok"
    except Exception as exc:  # surfaced by the parent
        results[rank] = repr(exc)
    finally:
        G.destroy_group()
        dist.destroy_process_group()


def test_public_api_on_two_gloo_ranks():
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}


def test_tiling_argument_is_checked(tmp_path):
    """``tiling=`` is honoured: the built tile shape passes, anything else is rejected (never silently ignored)."""
    import json

    from deepep_b200.ops import ep_gmm_fused as G

    shape = G.load_tiling_config()
    assert shape == {"m": 256, "n": 256, "k": 64}
    G._check_tiling(None)
    G._check_tiling({"m": 256})
    with pytest.raises(ValueError, match="not available"):
        G._check_tiling({"m": 128, "n": 256})
    with pytest.raises(ValueError, match="unknown tiling keys"):
        G._check_tiling({"rows": 256})
    with pytest.raises(TypeError):
        G._check_tiling([256, 256, 64])
    good, bad = tmp_path / "good.json", tmp_path / "bad.json"
    good.write_text(json.dumps(shape))
    bad.write_text(json.dumps({"k": 128}))
    assert G.load_tiling_config(good) == shape
    with pytest.raises(ValueError):
        G.load_tiling_config(bad)


def test_one_process_round_trip_and_every_rejection():
    """World size 1 on the CPU engine: both operators against the restatement, then every argument rule."""
    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    E, K, N = 3, 64, 128
    counts = [4, 0, 6]
    gen = torch.Generator().manual_seed(5)
    x = torch.randn((10, K), generator=gen).bfloat16()
    w = (torch.randn((E, K, N), generator=gen) / 8).bfloat16()
    with pytest.raises(RuntimeError, match="not initialised"):
        G.symmetric_input(4, K)
    with pytest.raises(ValueError, match="multiples of 64"):
        G.init_group(None, max_rows=16, max_k=K, max_n=100)
    cfg = G.init_group(None, max_rows=16, max_k=N, max_n=N)
    try:
        assert (cfg.rank, cfg.world_size, cfg.backend) == (0, 1, "cpu")
        with pytest.raises(RuntimeError, match="already initialised"):
            G.init_group(None, max_rows=16, max_k=K, max_n=N)
        assert G.symmetric_input(10, K).shape == (10, K) and G.symmetric_output(10, N).dtype == torch.bfloat16
        G.check_errors()                                               # nothing to check without device kernels
        out = G.all_to_allv_grouped_matmul(x, w, counts, torch.tensor(counts), ep_size=1, expert_num=E)
        ref, gathered = G.reference_alltoallv_gmm([x], [w], [counts], E)
        assert torch.equal(out, ref[0]) and torch.equal(gathered[0], x)
        w2 = (torch.randn((E, N, K), generator=gen) / 8).bfloat16()
        given = torch.empty((10, K), dtype=torch.bfloat16)
        back = G.grouped_matmul_all_to_allv(out, w2, counts, counts, ep_size=1, expert_num=E, out=given)
        assert back is given and torch.equal(back, G.reference_gmm_alltoallv([out], [w2], [counts], E)[0])
        a2a = lambda *a, **k: G.alltoallv_gmm(*a, **{**dict(ep_size=1, expert_num=E), **k})
        g2a = lambda *a, **k: G.gmm_alltoallv(*a, **{**dict(ep_size=1, expert_num=E), **k})
        for call, kind, message in (
                (lambda: a2a(x, w, counts, counts, ep_size=2), ValueError, "ep_size == group world_size"),
                (lambda: a2a(x, w, counts, counts, expert_num=0), ValueError, "divisible"),
                (lambda: a2a(x.float(), w, counts, counts), TypeError, "bf16"),
                (lambda: a2a(x, w[0], counts, counts), ValueError, "contiguous"),
                (lambda: a2a(x, w[:2], counts, counts), ValueError, "expert_num / ep_size"),
                (lambda: a2a(x[:, :32].contiguous(), w[:, :32].contiguous(), counts, counts), ValueError, "multiples of 64"),
                (lambda: a2a(x, w, counts[:2], counts), ValueError, "expert_num=3 elements"),
                (lambda: a2a(x, w, [4, -1, 7], counts), ValueError, "negative"),
                (lambda: a2a(x, w, torch.tensor([[4, 0, 6]]), counts), ValueError, "flat tensor"),
                (lambda: a2a(x, w, torch.tensor([4.0, 0.0, 6.0]), counts), TypeError, "int64 or int32"),
                (lambda: a2a(x, w, [4, 0, 5], counts), ValueError, "must equal x.shape"),
                (lambda: a2a(x, w, counts, counts, received_rows=-1), ValueError, "out of range"),
                (lambda: a2a(x, w, counts, counts, received_rows=9), ValueError, "does not match"),
                (lambda: a2a(x, w, counts, counts, all_to_allv_out=torch.empty((10, K), dtype=torch.bfloat16)), ValueError,
                 "requires output_all_to_allv"),
                (lambda: a2a(x, w, counts, counts, out=torch.empty((9, N), dtype=torch.bfloat16)), ValueError, "received_rows, n"),
                (lambda: a2a(x, w, counts, counts, output_all_to_allv=True, all_to_allv_out=torch.empty((10, K + 64), dtype=torch.bfloat16)),
                 ValueError, "all_to_allv_out must have shape"),
                (lambda: g2a(out, w2, counts, [4, 0, 5]), ValueError, "must equal x.shape"),
                (lambda: g2a(out, w2, counts, counts, out=torch.empty((10, K), dtype=torch.float32)), ValueError, "contiguous bf16"),
                (lambda: g2a(out, w2, counts, counts, out=torch.empty((9, K), dtype=torch.bfloat16)), ValueError,
                 "sum\\(local_tokens_per_expert\\), n")):
            with pytest.raises(kind, match=message):
                call()
        big = torch.zeros((17, K), dtype=torch.bfloat16)
        with pytest.raises(ValueError, match="at most 16"):
            a2a(big, w, [17, 0, 0], [17, 0, 0])
        with pytest.raises(ValueError, match="at most 16"):
            g2a(torch.zeros((17, N), dtype=torch.bfloat16), w2, [17, 0, 0], [17, 0, 0])
    finally:
        G.destroy_group()
    G.destroy_group()                                                  # idempotent
