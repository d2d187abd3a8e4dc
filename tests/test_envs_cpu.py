"""Upstream DeepEP's spawn helpers (``deep_ep.utils.envs``): ``init_dist`` joins a job as one of the local ranks of a
node, seeds the generators per rank and returns ``(rank, world, group)``; ``dist_print`` prints once per node.  Two CPU
processes (Gloo), then a dispatch / combine through the returned group.  Parity: ``deep_ep/utils/envs.py:55-101``."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(local_rank, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE="1", RANK="0")      # one node, two local ranks
    import deep_ep
    from deep_ep.utils import envs

    checks = {}
    try:
        with pytest.raises(RuntimeError, match="init_dist must be called"):
            envs.dist_print("too early")
        rank, world, group = envs.init_dist(local_rank, 2, seed=11)
        checks["identity"] = (rank, world) == (local_rank, 2) and os.environ["LOCAL_RANK"] == str(local_rank)
        checks["seeds"] = envs.get_global_seed() == 11 and envs.get_local_seed() == 11 + rank
        first = torch.rand(1).item()
        torch.manual_seed(11 + rank)
        checks["seeded"] = first == torch.rand(1).item()
        checks["domains"] = envs.get_physical_domain_size(group) == (1, 2) and envs.get_logical_domain_size(group) == (1, 2)
        envs.check_nvlink_connections(group)
        envs.dist_print(f"hello from {rank}", once_in_node=True)
        with pytest.raises(RuntimeError, match="already initialized"):
            envs.init_dist(local_rank, 2)
        buf = deep_ep.ElasticBuffer(group, num_max_tokens_per_rank=16, hidden=64, num_topk=2, explicitly_destroy=True)
        x = torch.randint(-3, 4, (10, 64)).to(torch.bfloat16)
        idx = torch.stack([torch.randperm(4)[:2] for _ in range(10)])
        rx, _, _, handle, _ = buf.dispatch(x, topk_idx=idx, num_experts=4, do_expand=True)
        out, _, _ = buf.combine(rx, handle)
        checks["round_trip"] = torch.equal(out.float(), x.float() * 2)
        buf.destroy()
    except Exception as exc:      # surfaced by the parent
        checks["error"] = repr(exc)
    finally:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
    results[local_rank] = checks


def test_init_dist_and_dist_print_on_two_local_ranks():
    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    port = _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(port, results), nprocs=2, join=True)
        got = dict(results)
    want = dict(identity=True, seeds=True, seeded=True, domains=True, round_trip=True)
    assert got == {0: want, 1: want}, got


def test_argument_rules_and_constants(monkeypatch):
    from deep_ep.utils import envs

    for args, kind in (((True, 2), TypeError), ((0, 2.0), TypeError), ((2, 2), ValueError), ((0, 0), ValueError)):
        with pytest.raises(kind):
            envs.init_dist(*args)
    monkeypatch.setenv("WORLD_SIZE", "2")
    monkeypatch.setenv("RANK", "5")
    with pytest.raises(ValueError, match="node-spawn"):
        envs.init_dist(0, 1)
    assert envs.get_nvlink_gbs() == pytest.approx(810.0) and envs.get_nvlink_gbs(1.0) == 900.0
    assert envs.get_rdma_gbs() == 0.0 and envs.check_fast_rdma_atomic_support() is False
    envs.check_torch_deterministic()
