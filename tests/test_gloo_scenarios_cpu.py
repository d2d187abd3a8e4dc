"""ElasticBuffer on four Gloo ranks against the all-rank oracle, bit for bit, over the routing scenarios of the device
tests (normal / random / invalid / empty / hotspot), both layouts, an aligned layout, fp8 pairs, uneven token counts and
an empty rank.  One process group serves all scenarios."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deepep_b200.oracle import reference as R
from helpers import bits_equal, make_routes, make_weights

WORLD, H, E, K = 4, 256, 16, 4
TOKENS = [40, 0, 17, 64]
SCENARIOS = [("normal", True, 1, False), ("random", True, 1, False), ("invalid", True, 8, False), ("empty", True, 1, False),
             ("hotspot", True, 1, False), ("random", False, 1, False), ("invalid", False, 1, False), ("random", True, 1, True)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(mode, seed):
    xs = [torch.randn((t, H), generator=torch.Generator().manual_seed(seed + r)).bfloat16() for r, t in enumerate(TOKENS)]
    idx = [make_routes(mode, t, E, K, WORLD, seed + 10 * r) for r, t in enumerate(TOKENS)]
    ws = [make_weights(t, K, seed + r) for r, t in enumerate(TOKENS)]
    return xs, idx, ws


def _worker(rank, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD, timeout=__import__("datetime").timedelta(seconds=120))
    from deepep_b200 import ElasticBuffer
    from deepep_b200.utils.math import per_token_cast_to_fp8

    buf = ElasticBuffer(dist.group.WORLD, num_max_tokens_per_rank=512, hidden=H, num_topk=K, explicitly_destroy=True)
    failures = []
    for n, (mode, expand, align, fp8) in enumerate(SCENARIOS):
        xs, idx, ws = _inputs(mode, 31 * n)
        send = [per_token_cast_to_fp8(x) for x in xs] if fp8 else xs
        ref, lays = R.dispatch(send, idx, ws, E, do_expand=expand, expert_alignment=align)
        rx, ridx, rw, handle, _ = buf.dispatch(send[rank], topk_idx=idx[rank], topk_weights=ws[rank], num_experts=E,
                                               do_expand=expand, expert_alignment=align if expand else None)
        want_x, want_idx, want_w = ref[rank]
        if fp8:
            good = bits_equal(rx[0], want_x[0]) and bits_equal(rx[1], want_x[1])
        else:
            good = bits_equal(rx, want_x)
        good = good and torch.equal(rw, want_w) and (expand or torch.equal(ridx, want_idx))
        good = good and handle.num_recv_tokens_per_expert_list == lays[rank].expert_counts.tolist()
        # combine: expert output = half of the received row; the value channel returns 0.5 - w per slot
        rows = [(o[0][0] if fp8 else o[0]) for o in ref]
        eouts = [torch.randn(r_.shape, generator=torch.Generator().manual_seed(5 + q)).bfloat16() if fp8
                 else (r_.float() * 0.5).bfloat16() for q, r_ in enumerate(rows)]
        evals = [0.5 - o[2] for o in ref]
        out, ow, _ = buf.combine(eouts[rank], handle, topk_weights=evals[rank])
        cref = R.combine(eouts, lays, TOKENS, K, topk_weights=evals)
        good = good and bits_equal(out, cref[rank][0]) and torch.equal(ow, cref[rank][1])
        if not good:
            failures.append((mode, expand, align, fp8))
    buf.destroy()
    results[rank] = failures
    dist.destroy_process_group()


def test_all_scenarios_on_four_gloo_ranks():
    port = _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(port, results), nprocs=WORLD, join=True)
        assert dict(results) == {r: [] for r in range(WORLD)}
