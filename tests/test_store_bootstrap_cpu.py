"""``ElasticBuffer`` without a process group: the ranks find each other through a TCPStore only.

Two forms: ``rank=`` / ``world_size=`` with ``bootstrap="store"`` (the store that a launcher serves on
``MASTER_ADDR:MASTER_PORT``), and an explicit :class:`StoreGroup` passed as ``group``.  Parity: the reference's
``StoreGroup`` bootstrap (``deep_ep/_store.py``, used where no ProcessGroup exists).  Two CPU processes, results
against the all-rank oracle; a disagreement between the ranks is reported by ``debug_collectives`` on both of them.
"""
import os
from datetime import timedelta

import pytest
import torch
import torch.multiprocessing as mp

from deepep_b200.oracle import reference as R
from helpers import bits_equal, make_routes, make_weights

WORLD, T, H, E, K = 2, [24, 9], 128, 8, 3


def _inputs():
    xs = [torch.randn((T[r], H), generator=torch.Generator().manual_seed(r)).bfloat16() for r in range(WORLD)]
    idx = [make_routes("invalid", T[r], E, K, WORLD, 20 + r) for r in range(WORLD)]
    ws = [make_weights(T[r], K, r) for r in range(WORLD)]
    return xs, idx, ws


def _worker(rank, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(WORLD))
    import deepep_b200 as deep_ep
    from deepep_b200.parallel.store import StoreGroup

    checks = {}
    try:
        xs, idx, ws = _inputs()
        ref, lays = R.dispatch(xs, idx, ws, E, do_expand=True)
        cref = R.combine([r[0] for r in ref], lays, T, K)
        buf = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=32, hidden=H, num_topk=K, explicitly_destroy=True,
                                    rank=rank, world_size=WORLD, bootstrap="store", device="cpu", debug_collectives=True,
                                    num_cpu_timeout_secs=60)
        checks["backend"] = buf.control.backend() == "store" and (buf.rank, buf.world_size) == (rank, WORLD)
        checks["machine"] = buf.machine_type == "cpu"
        rx, _, rw, handle, _ = buf.dispatch(xs[rank], topk_idx=idx[rank], topk_weights=ws[rank], num_experts=E, do_expand=True)
        checks["dispatch"] = bits_equal(rx, ref[rank][0]) and bits_equal(rw, ref[rank][2])
        out, _, _ = buf.combine(rx, handle)
        checks["combine"] = bits_equal(out, cref[rank][0])
        # the ranks make different calls: both learn of it before anything is exchanged
        try:
            buf.dispatch(xs[rank], topk_idx=idx[rank], topk_weights=ws[rank], num_experts=E, do_expand=(rank == 0))
            checks["disagreement"] = False
        except RuntimeError as exc:
            checks["disagreement"] = "disagree" in str(exc)
        buf.destroy()
        # an explicit StoreGroup as the group; a second group of the same job and prefix gets a session of its own
        group = StoreGroup.from_env(timeout=30)
        buf2 = deep_ep.ElasticBuffer(group, num_max_tokens_per_rank=32, hidden=H, num_topk=K, explicitly_destroy=True, device="cpu")
        rx2, ridx2, _, h2, _ = buf2.dispatch(xs[rank], topk_idx=idx[rank], num_experts=E)
        ref2, _ = R.dispatch(xs, idx, None, E, do_expand=False)
        checks["store_group"] = bits_equal(rx2, ref2[rank][0]) and torch.equal(ridx2, ref2[rank][1])
        buf2.destroy()
        group.close()
    except Exception as exc:          # surfaced by the parent
        checks["error"] = repr(exc)
    results[rank] = checks


def test_ranks_meet_through_a_store_only():
    from torch.distributed import TCPStore

    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    server = TCPStore("127.0.0.1", 0, None, True, timedelta(seconds=60), wait_for_workers=False)   # what a launcher serves
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(server.port, results), nprocs=WORLD, join=True)
        got = dict(results)
    for rank in range(WORLD):
        assert got[rank] == dict(backend=True, machine=True, dispatch=True, combine=True, disagreement=True, store_group=True), got


def test_a_rank_that_never_joins_ends_the_host_wait(monkeypatch):
    """``num_cpu_timeout_secs`` bounds the host-side waits of the bootstrap: with a peer that never shows up the
    constructor raises after about that long instead of waiting for ever (the failure is made on the host)."""
    import time

    from torch.distributed import TCPStore

    import deepep_b200 as deep_ep

    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    server = TCPStore("127.0.0.1", 0, None, True, timedelta(seconds=60), wait_for_workers=False)
    for name, value in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", str(server.port)), ("RANK", "0"), ("WORLD_SIZE", "2")):
        monkeypatch.setenv(name, value)
    started = time.monotonic()
    with pytest.raises(TimeoutError, match="did not appear"):
        deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=8, hidden=64, num_topk=2, rank=0, world_size=2, bootstrap="store",
                              device="cpu", num_cpu_timeout_secs=2)
    assert time.monotonic() - started < 30
