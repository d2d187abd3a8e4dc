"""Process-group bring-up helpers (one process per GPU, NCCL or Gloo).

Parity: ``deep_ep/utils/envs.py`` of the reference (``init_dist`` :55-101,
``init_seed`` :27-34, ``dist_print`` :45-52, domain sizes :104-118,
``get_nvlink_gbs`` :129-133 which returns 0 there; here it returns the
NVLink 5 per-direction figure scaled by ``factor``).
"""
from __future__ import annotations

import os
import random
from functools import lru_cache
from typing import Optional, Tuple

import torch
import torch.distributed as dist

_local_rank: Optional[int] = None
_local_seed: Optional[int] = None
_global_seed: Optional[int] = None

NVLINK5_GBS_PER_DIRECTION = 900.0


def init_seed(global_seed: int) -> None:
    global _local_seed, _global_seed
    _global_seed = global_seed
    _local_seed = global_seed + (dist.get_rank() if dist.is_initialized() else 0)
    torch.manual_seed(_local_seed)
    random.seed(_local_seed)


def get_local_seed() -> Optional[int]:
    return _local_seed


def get_global_seed() -> Optional[int]:
    return _global_seed


def dist_print(value: str = "", once_in_node: bool = False) -> None:
    if _local_rank is None:
        raise RuntimeError("init_dist must be called before dist_print")
    if not once_in_node or _local_rank == 0:
        print(value, flush=True)
    dist.barrier()


def init_dist(local_rank: int, num_local_ranks: int, seed: int = 0, backend: Optional[str] = None
              ) -> Tuple[int, int, "dist.ProcessGroup"]:
    """Join the job as ``local_rank`` of ``num_local_ranks`` processes on this node.

    ``WORLD_SIZE``/``RANK`` name the node count and node index, as in upstream
    DeepEP's spawn helpers.  ``backend`` defaults to NCCL when CUDA exists.
    """
    if not isinstance(local_rank, int) or isinstance(local_rank, bool):
        raise TypeError("local_rank must be an integer")
    if not isinstance(num_local_ranks, int) or isinstance(num_local_ranks, bool):
        raise TypeError("num_local_ranks must be an integer")
    if num_local_ranks <= 0 or not 0 <= local_rank < num_local_ranks:
        raise ValueError("local_rank must be in [0, num_local_ranks)")
    if dist.is_initialized():
        raise RuntimeError("torch.distributed is already initialized")
    addr = os.getenv("MASTER_ADDR", "127.0.0.1")
    port = int(os.getenv("MASTER_PORT", "8361"))
    nodes, node = int(os.getenv("WORLD_SIZE", "1")), int(os.getenv("RANK", "0"))
    if nodes <= 0 or not 0 <= node < nodes:
        raise ValueError("RANK must be in [0, WORLD_SIZE) for node-spawn mode")
    world, rank = nodes * num_local_ranks, node * num_local_ranks + local_rank
    global _local_rank
    _local_rank = local_rank
    os.environ["LOCAL_RANK"] = str(local_rank)
    use_cuda = torch.cuda.is_available()
    backend = backend or ("nccl" if use_cuda else "gloo")
    kwargs = dict(backend=backend, init_method=f"tcp://{addr}:{port}", world_size=world, rank=rank)
    if use_cuda:
        torch.cuda.set_device(local_rank)
        if backend == "nccl":
            kwargs["device_id"] = torch.device(f"cuda:{local_rank}")
    dist.init_process_group(**kwargs)
    init_seed(seed)
    return rank, world, dist.new_group(list(range(world)))


def get_physical_domain_size(group) -> Tuple[int, int]:
    """(scale-out domains, ranks per NVLink domain): one NVSwitch domain holds the group."""
    return 1, dist.get_world_size(group)


def get_logical_domain_size(group, allow_hybrid_mode: bool = True) -> Tuple[int, int]:
    del allow_hybrid_mode
    return 1, dist.get_world_size(group)


def check_nvlink_connections(group) -> None:
    """Every pair of GPUs in the group must be able to map each other's memory."""
    if not torch.cuda.is_available():
        return
    me = torch.cuda.current_device()
    for other in range(torch.cuda.device_count()):
        if other != me and not torch.cuda.can_device_access_peer(me, other):
            raise RuntimeError(f"GPU {me} cannot access GPU {other} as a peer")


def check_torch_deterministic() -> None:
    if torch.are_deterministic_algorithms_enabled() and torch.utils.deterministic.fill_uninitialized_memory:
        raise AssertionError("deterministic algorithms and fill_uninitialized_memory cannot both be enabled")


@lru_cache()
def get_nvlink_gbs(factor: float = 0.9) -> float:
    return NVLINK5_GBS_PER_DIRECTION * factor


@lru_cache()
def check_fast_rdma_atomic_support(nic_name: str = "") -> bool:
    del nic_name
    return False


@lru_cache()
def get_rdma_gbs(nic_name: str = "") -> float:
    del nic_name
    return 0.0


__all__ = [
    "check_fast_rdma_atomic_support", "check_nvlink_connections", "check_torch_deterministic", "dist_print",
    "get_global_seed", "get_local_seed", "get_logical_domain_size", "get_nvlink_gbs",
    "get_physical_domain_size", "get_rdma_gbs", "init_dist", "init_seed",
]
