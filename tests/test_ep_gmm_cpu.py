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
