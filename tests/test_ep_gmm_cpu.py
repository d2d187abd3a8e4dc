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
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=__import__("datetime").timedelta(seconds=120))
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


def test_balanced_route_builders():
    """Every source sends ``m`` rows, every destination receives ``m`` rows, neighbours differ by at most one row, and the
    per-rank tables are the matrix's row and column block (values for 7 rows over 2 ranks x 2 experts worked out by hand)."""
    assert G.build_global_route_matrix(7, 2, 4) == [[2, 2, 1, 2], [1, 2, 2, 2]]
    assert G.build_rank_route_tables(7, 1, 2, 4) == ([1, 2, 2, 2], [1, 2, 2, 2])
    for m, ep, experts in ((1, 1, 1), (4096, 4, 8), (4097, 8, 256), (13, 8, 8), (5, 4, 64)):
        matrix = torch.tensor(G.build_global_route_matrix(m, ep, experts))
        L = experts // ep
        assert matrix.shape == (ep, experts) and bool((matrix.sum(1) == m).all())
        per_destination = matrix.view(ep, ep, L).sum((0, 2))
        assert bool((per_destination == m).all())
        pairs = matrix.view(ep, ep, L)
        assert int(pairs.sum(2).max() - pairs.sum(2).min()) <= 1 and int((pairs.max(2).values - pairs.min(2).values).max()) <= 1
        for rank in range(ep):
            local, received = G.build_rank_route_tables(m, rank, ep, experts)
            assert local == matrix[rank].tolist() and received == matrix[:, rank * L:(rank + 1) * L].reshape(-1).tolist()
    lt, gt, rows = G.build_rank_route(100, 2, 4, 8, "cpu")
    assert lt.dtype == torch.int64 and gt.dtype == torch.int64 and rows == 100 == int(gt.sum()) == int(lt.sum())
    a, b = G.build_rank_route_tensors(100, 2, 4, 8, "cpu")
    assert torch.equal(a, lt) and torch.equal(b, gt)
    for args, message in (((0, 2, 4), "positive"), ((8, 9, 9), "exceed 8"), ((8, 2, 5), "divisible"), ((8, 1, 65), "exceed 64")):
        with pytest.raises(ValueError, match=message):
            G.build_global_route_matrix(*args)
    with pytest.raises(ValueError, match="rank must be"):
        G.build_rank_route_tables(8, 2, 2, 4)


def test_group_given_in_bytes_and_the_context_manager():
    """The reference's forms: ``with udma_group(...)`` and ``init_udma_group(heap_size=...)``; the workspace is sized by
    the first operator call.  One process, CPU engine."""
    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    E, K, N, m = 4, 64, 128, 24
    gen = torch.Generator().manual_seed(2)
    x = torch.randn((m, K), generator=gen).bfloat16()
    w1 = (torch.randn((E, K, N), generator=gen) / 8).bfloat16()
    w2 = (torch.randn((E, N, K), generator=gen) / 8).bfloat16()
    local_counts, received_counts, rows = G.build_rank_route(m, 0, 1, E, "cpu")
    with G.udma_group(heap_size=2 << 20) as cfg:
        assert cfg.world_size == 1 and G.get_udma_config().backend == "pending"
        with G.udma_group():                                            # nested: borrows, does not destroy on exit
            h = G.alltoallv_gmm(x, w1, local_counts, received_counts, ep_size=1, expert_num=E, received_rows=rows)
        sized = G.get_udma_config()
        assert isinstance(sized, G.UdmaConfig) and (sized.max_k, sized.max_n) == (128, 128) and sized.max_rows == (2 << 20) // 512
        y = G.gmm_alltoallv(h, w2, local_counts, received_counts, ep_size=1, expert_num=E)
        with pytest.raises(RuntimeError, match="contexts are active"):
            G.destroy_udma_group()
    with pytest.raises(RuntimeError, match="not initialised"):
        G.get_udma_config()                                              # the outermost context destroyed what it created
    ref_h, _ = G.reference_alltoallv_gmm([x], [w1], [local_counts.tolist()], E)
    assert torch.equal(h, ref_h[0]) and torch.equal(y, G.reference_gmm_alltoallv([h], [w2], [local_counts.tolist()], E)[0])
    # an explicitly initialised group is borrowed by a context and survives it
    G.init_udma_group(rank=0, world_size=1, heap_size=1 << 20, init_method="tcp://127.0.0.1:1")
    try:
        with G.udma_group():
            assert G.symmetric_input(4, K).shape == (4, K)               # sizes the workspace for this width
        assert G.get_udma_config().max_k == 64
        with pytest.raises(RuntimeError, match="already initialised"):
            G.init_udma_group(heap_size=1 << 20)
    finally:
        G.destroy_udma_group()
    with pytest.raises(ValueError, match="together"):
        G.init_group(None, max_rows=8)
    with pytest.raises(ValueError, match="1 MiB"):
        G.init_udma_group(heap_size=1000)
