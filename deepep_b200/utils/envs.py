"""Bringing up a job of one process per GPU, and what the machine offers it.

The functions carry the names that test and benchmark programs written for upstream DeepEP call (parity:
``deep_ep/utils/envs.py`` of the reference: ``init_dist``, ``init_seed``, ``dist_print``, the domain sizes, the link
figures).  The answers are those of one NVSwitch domain of B200s: every rank is an NVLink peer of every other, there
is no scale-out network, and the link figure is NVLink 5's 900 GB/s per direction (the reference reports 0 there,
having no such link).
"""
from __future__ import annotations

import dataclasses
import os
import random
from typing import Optional, Tuple

import torch
import torch.distributed as dist

NVLINK5_GBS_PER_DIRECTION = 900.0


@dataclasses.dataclass
class _Job:
    """What this process learnt when it joined: its index on the node and the seeds it drew."""
    local_rank: Optional[int] = None
    global_seed: Optional[int] = None
    local_seed: Optional[int] = None


_JOB = _Job()


def _plain_int(value, name: str) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise TypeError(f"{name} must be an integer")
    return value


def _placement(local_rank: int, num_local_ranks: int) -> Tuple[int, int]:
    """``(rank, world)`` of process ``local_rank`` when ``WORLD_SIZE`` counts nodes and ``RANK`` names this node (the
    convention of upstream's spawn helpers: one launcher per node, ``num_local_ranks`` children each)."""
    nodes, node = int(os.getenv("WORLD_SIZE", "1")), int(os.getenv("RANK", "0"))
    if nodes <= 0 or not 0 <= node < nodes:
        raise ValueError("RANK must be in [0, WORLD_SIZE) for node-spawn mode")
    return node * num_local_ranks + local_rank, nodes * num_local_ranks


def init_seed(global_seed: int) -> None:
    """Seed torch and ``random`` with ``global_seed + rank`` so that the ranks draw different data reproducibly."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    _JOB.global_seed, _JOB.local_seed = global_seed, global_seed + rank
    random.seed(_JOB.local_seed)
    torch.manual_seed(_JOB.local_seed)


def get_local_seed() -> Optional[int]:
    return _JOB.local_seed


def get_global_seed() -> Optional[int]:
    return _JOB.global_seed


def init_dist(local_rank: int, num_local_ranks: int, seed: int = 0, backend: Optional[str] = None
              ) -> Tuple[int, int, "dist.ProcessGroup"]:
    """Join the job as child ``local_rank`` of ``num_local_ranks`` on this node; returns ``(rank, world, group)``.

    The rendezvous is ``tcp://MASTER_ADDR:MASTER_PORT`` (127.0.0.1:8361 when unset).  With CUDA the process takes GPU
    ``local_rank`` and NCCL is bound to it at once (``device_id``), so the first collective does not pay for a lazy
    communicator; without CUDA, or with ``backend="gloo"``, the same call brings up a CPU job.
    """
    local_rank, num_local_ranks = _plain_int(local_rank, "local_rank"), _plain_int(num_local_ranks, "num_local_ranks")
    if num_local_ranks <= 0 or not 0 <= local_rank < num_local_ranks:
        raise ValueError("local_rank must be in [0, num_local_ranks)")
    if dist.is_initialized():
        raise RuntimeError("torch.distributed is already initialized")
    rank, world = _placement(local_rank, num_local_ranks)
    on_gpu = torch.cuda.is_available()
    chosen = backend if backend else ("nccl" if on_gpu else "gloo")
    binding = {}
    if on_gpu:
        torch.cuda.set_device(local_rank)
        if chosen == "nccl":
            binding["device_id"] = torch.device("cuda", local_rank)
    os.environ["LOCAL_RANK"] = str(local_rank)
    _JOB.local_rank = local_rank
    endpoint = "tcp://{}:{}".format(os.getenv("MASTER_ADDR", "127.0.0.1"), int(os.getenv("MASTER_PORT", "8361")))
    dist.init_process_group(chosen, init_method=endpoint, rank=rank, world_size=world, **binding)
    init_seed(seed)
    return rank, world, dist.new_group(list(range(world)))


def dist_print(value: str = "", once_in_node: bool = False) -> None:
    """Print on every rank (or on the first rank of each node only), then meet at a barrier so output stays grouped."""
    if _JOB.local_rank is None:
        raise RuntimeError("init_dist must be called before dist_print")
    if _JOB.local_rank == 0 or not once_in_node:
        print(value, flush=True)
    dist.barrier()


def get_physical_domain_size(group) -> Tuple[int, int]:
    """``(scale-out domains, ranks per NVLink domain)``: the whole group sits in one NVSwitch domain."""
    return 1, dist.get_world_size(group)


def get_logical_domain_size(group, allow_hybrid_mode: bool = True) -> Tuple[int, int]:
    """Same as the physical sizes; there is no second network to run a hybrid mode over."""
    return get_physical_domain_size(group)


def check_nvlink_connections(group) -> None:
    """Raise unless this process's GPU can map the memory of every other GPU of the machine."""
    if not torch.cuda.is_available():
        return
    mine = torch.cuda.current_device()
    unreachable = [other for other in range(torch.cuda.device_count())
                   if other != mine and not torch.cuda.can_device_access_peer(mine, other)]
    if unreachable:
        raise RuntimeError(f"GPU {mine} cannot access GPU {unreachable[0]} as a peer")


def check_torch_deterministic() -> None:
    """Buffers here are taken with ``torch.empty`` and filled by kernels; torch's deterministic mode with
    ``fill_uninitialized_memory`` would add a fill to every one of them, so that combination is refused."""
    if torch.are_deterministic_algorithms_enabled() and torch.utils.deterministic.fill_uninitialized_memory:
        raise AssertionError("deterministic algorithms and fill_uninitialized_memory cannot both be enabled")


def get_nvlink_gbs(factor: float = 0.9) -> float:
    """NVLink 5 bandwidth per direction per GPU in GB/s, scaled by ``factor`` (what a copy can hope to reach)."""
    return factor * NVLINK5_GBS_PER_DIRECTION


def check_fast_rdma_atomic_support(nic_name: str = "") -> bool:
    """No scale-out NIC takes part: always ``False``."""
    return False


def get_rdma_gbs(nic_name: str = "") -> float:
    """No scale-out NIC takes part: 0 GB/s."""
    return 0.0


__all__ = [
    "check_fast_rdma_atomic_support", "check_nvlink_connections", "check_torch_deterministic", "dist_print",
    "get_global_seed", "get_local_seed", "get_logical_domain_size", "get_nvlink_gbs",
    "get_physical_domain_size", "get_rdma_gbs", "init_dist", "init_seed",
]
