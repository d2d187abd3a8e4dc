"""Process-level runtime: control plane, native session, comm stream, lifecycle.

Parity: ``deep_ep/_runtime.py:67-290`` of the reference (``Runtime``: capacity
and timeout validation, cross-rank agreement on the configuration vector,
exchange of the workspace identity, creation of the communication stream and
of the native session, ``barrier``, ``close``, poisoning after a failed
launch, ``ResourceWarning`` for buffers that were never destroyed).
Here the identity that ranks exchange is a CUDA IPC handle of the workspace.
"""
from __future__ import annotations

import os
import warnings
from typing import Any, List, Optional

import torch

from .store import StoreGroup


class ControlPlane:
    """Small host-collective interface with three backends: ProcessGroup, TCPStore, single process."""

    def __init__(self, group: Any = None, rank: Optional[int] = None, world_size: Optional[int] = None,
                 bootstrap: str = "default"):
        import torch.distributed as dist

        self.group, self.store = None, None
        if isinstance(group, StoreGroup):
            self.store, self.rank, self.size = group, group.rank(), group.size()
        elif group is not None:
            self.group, self.rank, self.size = group, dist.get_rank(group), dist.get_world_size(group)
        elif world_size in (None, 1) and rank in (None, 0) and bootstrap != "store":
            if dist.is_initialized() and world_size is None:
                self.group, self.rank, self.size = dist.group.WORLD, dist.get_rank(), dist.get_world_size()
            else:
                self.rank, self.size = 0, 1
        else:
            if rank is None or world_size is None:
                raise ValueError("rank= and world_size= are both required when no group is given")
            os.environ.setdefault("RANK", str(rank))
            os.environ.setdefault("WORLD_SIZE", str(world_size))
            self.store = StoreGroup.from_env()
            self.rank, self.size = rank, world_size
        if rank is not None and rank != self.rank:
            raise ValueError(f"rank={rank} contradicts the group's rank {self.rank}")
        if world_size is not None and world_size != self.size:
            raise ValueError(f"world_size={world_size} contradicts the group's size {self.size}")

    def all_gather_object(self, obj: Any) -> List[Any]:
        import torch.distributed as dist

        if self.size == 1:
            return [obj]
        if self.group is not None:
            out = [None] * self.size
            dist.all_gather_object(out, obj, group=self.group)
            return out
        import base64
        import pickle

        raw = self.store.all_gather(base64.b64encode(pickle.dumps(obj)).decode("ascii"), "object")
        return [pickle.loads(base64.b64decode(r)) for r in raw]

    def barrier(self) -> None:
        import torch.distributed as dist

        if self.size == 1:
            return
        if self.group is not None:
            dist.barrier(group=self.group)
        else:
            self.store.barrier()

    def backend(self) -> str:
        import torch.distributed as dist

        if self.group is not None:
            return dist.get_backend(self.group)
        return "store" if self.store is not None else "single"


_busy_runtimes = 0


class Runtime:
    """Owns the native session of this process for one buffer."""

    def __init__(self, control: ControlPlane, layout, timeout: float, device: torch.device):
        from ..ops import require_native

        global _busy_runtimes
        self.C = require_native("shared-memory runtime")
        self.control, self.layout, self.device = control, layout, device
        self.rank, self.world = control.rank, control.size
        if not 1 <= timeout <= 3600:
            raise ValueError("num_gpu_timeout_secs must be in [1, 3600]")
        self.failed = False
        self.closed = False
        # every rank must ask for the same workspace
        config = [int(layout.total), int(layout.max_tokens), int(layout.hidden), int(layout.topk), int(timeout), self.world]
        configs = control.all_gather_object(config)
        if any(c != configs[0] for c in configs):
            raise RuntimeError(f"ranks disagree on the buffer configuration: {configs}")
        torch.cuda.set_device(device)
        error, handle = None, None
        try:
            self.native = self.C.Session(self.rank, self.world, layout.total, float(timeout))
            handle = bytes(self.native.ipc_handle()) if self.world > 1 else b""
        except Exception as exc:  # tell the peers before raising, so nobody waits for a handle
            error = repr(exc)
        replies = control.all_gather_object((error, handle))
        errors = [f"rank {r}: {e}" for r, (e, _) in enumerate(replies) if e]
        if errors:
            if error is None:
                self.native.close()
            raise RuntimeError("workspace creation failed: " + "; ".join(errors))
        if self.world > 1:
            self.native.open_peers([h for _, h in replies])
        if not self.native.mapped():
            raise RuntimeError("a peer workspace is not mapped")
        self.stream = torch.cuda.Stream(device=device)
        control.barrier()
        _busy_runtimes += 1

    def ensure_alive(self) -> None:
        if self.closed:
            raise RuntimeError("the buffer was destroyed")
        if self.failed or self.native.poisoned:
            raise RuntimeError("A previous communication launch failed; restart the distributed job")

    def close(self) -> None:
        global _busy_runtimes
        if self.closed:
            return
        torch.cuda.synchronize(self.device)
        self.control.barrier()   # nobody may still be writing into a workspace that is about to be freed
        try:
            if not self.native.guard_intact():      # the canary zone behind the workspace (peers map it as well)
                warnings.warn("something wrote behind this rank's symmetric workspace; results of this buffer are suspect",
                              RuntimeWarning)
        except RuntimeError:
            pass
        try:
            self.native.close()
        finally:
            self.closed = True
            _busy_runtimes -= 1
        self.control.barrier()

    def __del__(self):
        if not getattr(self, "closed", True):
            warnings.warn("ElasticBuffer was never destroyed; call destroy() on every rank", ResourceWarning)


def runtime_busy() -> bool:
    return _busy_runtimes > 0
