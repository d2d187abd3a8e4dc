"""alltoallv_gmm / gmm_alltoallv kernels (virtual ranks in one cooperative launch) against a plain fp32 restatement."""
import pytest
import torch

from deepep_b200.ops import ep_gmm_fused as G

pytestmark = pytest.mark.gpu


def _counts(world, E, max_rows, seed, empty_expert=None):
    g = torch.Generator().manual_seed(seed)
    out = []
    for s in range(world):
        c = torch.randint(0, 2 * max_rows // E + 1, (E,), generator=g)
        if empty_expert is not None:
            c[empty_expert] = 0
        while int(c.sum()) > max_rows:
            c = c // 2
        out.append(c.tolist())
    return out


def _close(actual, expected, what):
    a, e = actual.float().cpu(), expected.float()
    assert a.shape == e.shape, (what, a.shape, e.shape)
    if a.numel() == 0:
        return
    err = (a - e).abs().max().item()
    scale = e.abs().max().item() + 1e-6
    assert err <= 2e-2 * scale, f"{what}: max abs error {err} against magnitude {scale}"


def _world(world, E, K, N, max_rows, seed=0, empty_expert=None, reps=2, zero_copy=False):
    from deepep_b200.ops import load_native

    C = load_native()
    dev = torch.device("cuda")
    L = E // world
    counts = _counts(world, E, max_rows, seed, empty_expert)
    gen = torch.Generator().manual_seed(seed + 1)
    xs = [torch.randn((sum(c), K), generator=gen).to(torch.bfloat16) for c in counts]
    ws = [(torch.randn((L, K, N), generator=gen) / K ** 0.5).to(torch.bfloat16) for _ in range(world)]
    ref_out, ref_gathered = G.reference_alltoallv_gmm(xs, ws, counts, E)
    # second op: the expert ranks multiply what they gathered by a second weight and send it back
    ws2 = [(torch.randn((L, K, N), generator=gen) / K ** 0.5).to(torch.bfloat16) for _ in range(world)]
    ref_back = G.reference_gmm_alltoallv(ref_gathered, ws2, counts, E)

    layout = C.make_mega_layout(world, 1, 128, 1, G.GmmEngine.region_bytes(C, max_rows, K, N))
    sessions = [C.Session(r, world, layout.total, 20.0) for r in range(world)]
    for s in sessions:
        s.attach_peers([q.workspace for q in sessions])
    try:
        eng = G.GmmEngine(sessions, layout, dev, max_rows, K, N)
        d_x = [x.to(dev) for x in xs]
        if zero_copy:    # inputs written into the stage area are read by the peers in place
            d_x = [eng.symmetric_input(r, x.shape[0], K) for r, x in enumerate(xs)]
            for v, x in zip(d_x, xs):
                v.copy_(x)
        d_w, d_w2 = [w.to(dev) for w in ws], [w.to(dev) for w in ws2]
        d_c = [torch.tensor(c, dtype=torch.int32, device=dev) for c in counts]
        for rep in range(reps):
            outs = [torch.full((r.shape[0], N), float("nan"), dtype=torch.bfloat16, device=dev) for r in ref_out]
            gath = [torch.full((r.shape[0], K), float("nan"), dtype=torch.bfloat16, device=dev) for r in ref_gathered]
            eng.a2av_gmm(d_x, d_w, d_c, outs, gath, num_experts=E)
            back = [torch.full((x.shape[0], N), float("nan"), dtype=torch.bfloat16, device=dev) for x in xs]
            if zero_copy:
                back = [eng.symmetric_output(r, x.shape[0], N) for r, x in enumerate(xs)]
            eng.gmm_a2av(gath, d_w2, d_c, back, num_experts=E)
            torch.cuda.synchronize()
            eng.check()
            for s in sessions:
                assert s.status()["code"] == 0, s.status()
            for r in range(world):
                assert torch.equal(gath[r].cpu(), ref_gathered[r]), f"rank {r}: gathered rows differ (rep {rep})"
                _close(outs[r], ref_out[r], f"a2av_gmm rank {r} rep {rep}")
                _close(back[r], ref_back[r], f"gmm_a2av rank {r} rep {rep}")
    finally:
        torch.cuda.synchronize()
        for s in sessions:
            s.close()


def test_single_rank_grouped_gemm():
    _world(1, 4, 256, 256, 600)


def test_two_ranks_odd_sizes():
    _world(2, 6, 192, 320, 500, seed=3, empty_expert=2)


def test_zero_copy_views():
    _world(2, 4, 128, 128, 400, seed=9, zero_copy=True)


def test_four_ranks():
    _world(4, 8, 512, 512, 700, seed=5)


def test_eight_ranks_many_experts():
    _world(8, 32, 128, 256, 300, seed=7, empty_expert=9)


def test_row_counts_that_do_not_fit_are_reported():
    from deepep_b200.ops import load_native

    C = load_native()
    dev = torch.device("cuda")
    E, K, N, max_rows = 2, 64, 64, 256
    layout = C.make_mega_layout(1, 1, 128, 1, G.GmmEngine.region_bytes(C, max_rows, K, N))
    s = C.Session(0, 1, layout.total, 20.0)
    s.attach_peers([s.workspace])
    try:
        eng = G.GmmEngine([s], layout, dev, max_rows, K, N)
        x = torch.zeros((100, K), dtype=torch.bfloat16, device=dev)
        w = torch.zeros((E, K, N), dtype=torch.bfloat16, device=dev)
        counts = torch.tensor([90, 90], dtype=torch.int32, device=dev)     # 180 rows claimed, 100 staged
        out = torch.zeros((180, N), dtype=torch.bfloat16, device=dev)
        eng.a2av_gmm([x], [w], [counts], [out], num_experts=E)
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="row counts"):
            eng.check()
    finally:
        s.close()


def _real_worker(rank, world, port, results):
    import os

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        E, K, N, max_rows = 8, 256, 320, 600
        L = E // world
        counts = _counts(world, E, max_rows, 21, empty_expert=3)
        gen = torch.Generator().manual_seed(22)
        xs = [torch.randn((sum(c), K), generator=gen).to(torch.bfloat16) for c in counts]
        ws = [(torch.randn((L, K, N), generator=gen) / K ** 0.5).to(torch.bfloat16) for _ in range(world)]
        ws2 = [(torch.randn((L, K, N), generator=gen) / K ** 0.5).to(torch.bfloat16) for _ in range(world)]
        ref_out, ref_g = G.reference_alltoallv_gmm(xs, ws, counts, E)
        ref_back = G.reference_gmm_alltoallv(ref_g, ws2, counts, E)
        G.init_group(dist.group.WORLD, max_rows=max_rows, max_k=K, max_n=N, timeout=30.0)
        glob = [counts[s][rank * L + l] for s in range(world) for l in range(L)]
        for rep in range(2):
            out, gathered = G.alltoallv_gmm(xs[rank].to(dev), ws[rank].to(dev), counts[rank], torch.tensor(glob, device=dev),
                                            ep_size=world, expert_num=E, output_all_to_allv=True)
            back = G.gmm_alltoallv(gathered, ws2[rank].to(dev), torch.tensor(counts[rank], device=dev), glob, ep_size=world, expert_num=E)
            torch.cuda.synchronize()
            assert torch.equal(gathered.cpu(), ref_g[rank])
            _close(out, ref_out[rank], f"a2av_gmm rank {rank} rep {rep}")
            _close(back, ref_back[rank], f"gmm_a2av rank {rank} rep {rep}")
        results[rank] = True
    except Exception as exc:  # surfaced by the parent
        results[rank] = repr(exc)
    finally:
        G.destroy_group()
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_real_ranks_public_api(world):
    import socket

    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    results = mp.Manager().dict()
    mp.spawn(_real_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {r: True for r in range(world)}
