"""The buffer self-checks used by the benchmarks: they pass on a correct buffer (Gloo, two CPU ranks) and catch damage."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import make_routes, make_weights


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=__import__("datetime").timedelta(seconds=120))
    import deepep_b200 as deep_ep
    from deepep_b200.utils import verify as V

    T, H, E, K = 96 + 8 * rank, 256, 16, 4
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(rank)).bfloat16()
    out = {}
    for mode in ("random", "invalid"):
        idx, w = make_routes(mode, T, E, K, world, 3 + rank), make_weights(T, K, rank)
        buf = deep_ep.ElasticBuffer(dist.group.WORLD, num_max_tokens_per_rank=512, hidden=H, num_topk=K, explicitly_destroy=True)
        out[mode] = V.verify_dispatch_combine(buf, x, idx, w, E)
        # damage: a combine that drops one row's contribution must be caught on the rank that owns the row
        real = buf.combine

        def broken(rows, handle, *a, **k):
            rows = rows.clone()
            rows[0] = 0
            return real(rows, handle, *a, **k)

        buf.combine = broken
        out[mode + "_broken"] = V.verify_dispatch_combine(buf, x, idx, w, E)
        buf.combine = real
        buf.destroy()
    small = deep_ep.ElasticBuffer(dist.group.WORLD, num_max_tokens_per_rank=128, hidden=H, num_topk=K, explicitly_destroy=True)
    idx, w = make_routes("random", T, E, K, world, 9 + rank), make_weights(T, K, 5 + rank)
    out["ll"] = V.verify_low_latency(small, x, idx, w, E)
    small.destroy()
    results[rank] = out
    dist.destroy_process_group()


def test_self_checks_pass_and_catch_damage():
    world, port = 2, _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        res = dict(results)
    for r in range(world):
        for mode in ("random", "invalid"):
            ok, details = res[r][mode]
            assert ok, (r, mode, details)
            ok, details = res[r][mode + "_broken"]
            assert not ok                                           # the verdict is agreed by all ranks
        ok, details = res[r]["ll"]
        assert ok, (r, details)
    assert any(not res[r]["random_broken"][1]["combine_ok"] for r in range(world))


def test_row_checksums_see_swapped_columns():
    from deepep_b200.utils.verify import row_checksums

    x = torch.randn(4, 64).bfloat16()
    y = x.clone()
    y[:, [0, 1]] = y[:, [1, 0]]
    a, b = row_checksums(x), row_checksums(y)
    assert torch.equal(a[:, 0], b[:, 0]) and not torch.equal(a[:, 1], b[:, 1])
