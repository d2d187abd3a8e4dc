"""The low-latency contract of ``ElasticBuffer`` on four Gloo ranks: a buffer of at most 256 tokens serves a default
fresh dispatch with weights on the decode path (expert-major rows, weights applied at the source in slot order), with the
same results as the all-rank oracle."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deepep_b200.oracle import reference as R
from helpers import bits_equal, make_routes, make_weights

WORLD, H, E, K = 4, 256, 32, 8
TOKENS = [128, 1, 0, 77]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD, timeout=__import__("datetime").timedelta(seconds=120))
    from deepep_b200 import ElasticBuffer

    buf = ElasticBuffer(dist.group.WORLD, num_max_tokens_per_rank=128, hidden=H, num_topk=K, explicitly_destroy=True)
    bad = []
    for rep, mode in enumerate(("random", "invalid", "hotspot")):
        xs = [torch.randn((t, H), generator=torch.Generator().manual_seed(9 * rep + r)).bfloat16() for r, t in enumerate(TOKENS)]
        idx = [make_routes(mode, t, E, K, WORLD, 5 * rep + r) for r, t in enumerate(TOKENS)]
        ws = [make_weights(t, K, rep + r) for r, t in enumerate(TOKENS)]
        ref, lays = R.dispatch(xs, idx, ws, E, do_expand=True)
        # the choice of path must not depend on a rank's own batch: the rank with no tokens takes the decode path too
        rx, _, rw, handle, _ = buf.dispatch(xs[rank], topk_idx=idx[rank], topk_weights=ws[rank], num_experts=E)
        low = handle.is_low_latency
        good = bits_equal(rx, ref[rank][0]) and torch.equal(rw, ref[rank][2])
        good = good and handle.num_recv_tokens_per_expert_list == lays[rank].expert_counts.tolist()
        eouts = [(o[0].float() * 0.25).bfloat16() for o in ref]
        if low:
            out, _, _ = buf.combine(eouts[rank], handle)
            good = good and bits_equal(out, R.low_latency_combine(eouts, lays, ws, TOKENS)[rank])
        bad.append((mode, low, good))
    buf.destroy()
    results[rank] = bad
    dist.destroy_process_group()


def test_low_latency_contract_on_gloo_ranks():
    port = _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(port, results), nprocs=WORLD, join=True)
        for rank in range(WORLD):
            assert all(good for _, _, good in results[rank]), (rank, results[rank])
            assert all(low for _, low, _ in results[rank]), (rank, results[rank])
