"""Process-level runtime: control plane, native session, comm stream, lifecycle.

Parity: ``deep_ep/_runtime.py:67-290`` of the reference (``Runtime``: capacity
and timeout validation, cross-rank agreement on the configuration vector,
exchange of the workspace identity, creation of the communication stream and
of the native session, ``barrier``, ``close``, poisoning after a failed
launch, ``ResourceWarning`` for buffers that were never destroyed).
The identity that ranks exchange is either a file descriptor of a CUDA
virtual-memory allocation, passed over Unix sockets (``vmm``), or a CUDA IPC
memory handle that travels through the control plane (``ipc``);
``DEEPEP_TRANSPORT=auto|vmm|ipc`` selects (``auto``: ``vmm`` when every rank's
driver supports it).
"""
from __future__ import annotations

import os
import warnings
from typing import Any, List, Optional

import torch

from .store import StoreGroup
from .streams import resolve_comm_stream


class ControlPlane:
    """Small host-collective interface with four backends: ProcessGroup, TCPStore, an MPI communicator, single process."""

    def __init__(self, group: Any = None, rank: Optional[int] = None, world_size: Optional[int] = None,
                 bootstrap: str = "default", timeout: float = 300.0):
        """``timeout`` (seconds) bounds the host-side waits this object owns: the operations of a store group it opens
        itself and the hand-over of file descriptors between the ranks."""
        import torch.distributed as dist

        self.group, self.store, self.mpi, self.timeout = None, None, None, float(timeout)
        if isinstance(group, StoreGroup):
            self.store, self.rank, self.size = group, group.rank(), group.size()
        elif all(hasattr(group, name) for name in ("Get_rank", "Get_size", "allgather", "Barrier")):
            # an MPI communicator (mpi4py): the reference's MPI bootstrap (``deep_ep/_runtime.py:94-104`` there)
            self.mpi, self.rank, self.size = group, int(group.Get_rank()), int(group.Get_size())
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
            self.store = StoreGroup.from_env(timeout=self.timeout)
            self.rank, self.size = rank, world_size
        if rank is not None and rank != self.rank:
            raise ValueError(f"rank={rank} contradicts the group's rank {self.rank}")
        if world_size is not None and world_size != self.size:
            raise ValueError(f"world_size={world_size} contradicts the group's size {self.size}")

    def all_gather_object(self, obj: Any) -> List[Any]:
        import torch.distributed as dist

        if self.size == 1:
            return [obj]
        if self.mpi is not None:
            return list(self.mpi.allgather(obj))
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
        if self.mpi is not None:
            self.mpi.Barrier()
        elif self.group is not None:
            dist.barrier(group=self.group)
        else:
            self.store.barrier()

    def backend(self) -> str:
        import torch.distributed as dist

        if self.mpi is not None:
            return "mpi"
        if self.group is not None:
            return dist.get_backend(self.group)
        return "store" if self.store is not None else "single"


_busy_runtimes = 0


def exchange_fds(control: ControlPlane, fd: int, timeout: Optional[float] = None) -> List[int]:
    """Every rank hands ``fd`` to every peer over Unix-domain sockets (SCM_RIGHTS); returns one descriptor per rank
    (``-1`` at this rank's own index).  The caller owns the returned descriptors.

    Each rank listens on an abstract socket whose name carries a token chosen by rank 0; a background thread serves
    ``size - 1`` connections while the rank itself collects the peers' descriptors one after the other.
    """
    import secrets
    import socket
    import threading

    rank, size = control.rank, control.size
    if size == 1:
        return [-1]
    timeout = min(60.0, getattr(control, "timeout", 60.0)) if timeout is None else timeout
    token = control.all_gather_object(secrets.token_hex(8) if rank == 0 else None)[0]
    name = lambda r: f"\0deepep-{token}-{r}"
    server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    server.bind(name(rank))
    server.listen(size)
    server.settimeout(timeout)
    errors: List[str] = []

    def serve():
        try:
            for _ in range(size - 1):
                conn, _addr = server.accept()
                with conn:
                    socket.send_fds(conn, [b"fd"], [fd])
        except Exception as exc:          # reported after the join below
            errors.append(repr(exc))

    thread = threading.Thread(target=serve, daemon=True)
    thread.start()
    control.barrier()                      # every listener is up
    out = [-1] * size
    try:
        for step in range(1, size):
            peer = (rank + step) % size
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as client:
                client.settimeout(timeout)
                client.connect(name(peer))
                _msg, fds, _flags, _addr = socket.recv_fds(client, 16, 1)
                if len(fds) != 1:
                    raise RuntimeError(f"rank {peer} sent no file descriptor")
                out[peer] = fds[0]
        thread.join(timeout)
        if errors or thread.is_alive():
            raise RuntimeError("handing the workspace descriptor to the peers failed: " + "; ".join(errors or ["timed out"]))
    except Exception:
        import os as _os

        for f in out:
            if f >= 0:
                _os.close(f)
        raise
    finally:
        server.close()
    return out


def shutdown_session(control: ControlPlane, native, synchronize=None) -> None:
    """Collective teardown of one workspace.  No rank frees its workspace while a peer still maps it: every rank
    drops its peer mappings, a barrier follows, and only then does each rank free its own allocation (freeing an
    exported allocation that an importer still has open is undefined)."""
    if synchronize is not None:
        synchronize()
    control.barrier()            # nobody is still writing into a workspace that is about to go away
    try:
        native.close_peers()
    finally:
        control.barrier()        # every peer mapping is gone
        native.close()
    control.barrier()


class Runtime:
    """Owns the native session of this process for one buffer."""

    def __init__(self, control: ControlPlane, layout, timeout: float, device: torch.device, comm_stream: Any = None):
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
        if device.type == "cuda":          # (a CPU device only occurs in tests that swap the CUDA entry points for doubles)
            torch.cuda.set_device(device)
        wanted = os.environ.get("DEEPEP_TRANSPORT", "auto").lower()
        if wanted not in ("auto", "vmm", "ipc"):
            raise ValueError("DEEPEP_TRANSPORT must be auto, vmm or ipc")
        # one transport for the whole job: virtual-memory allocations only when every rank can share them
        votes = control.all_gather_object((wanted, bool(self.C.vmm_supported())))
        if any(v[0] != wanted for v in votes):
            raise RuntimeError(f"ranks disagree on DEEPEP_TRANSPORT: {[v[0] for v in votes]}")
        if wanted == "vmm" and not all(v[1] for v in votes):
            raise RuntimeError("DEEPEP_TRANSPORT=vmm, but a rank's driver cannot share virtual-memory allocations")
        self.transport = "vmm" if wanted != "ipc" and all(v[1] for v in votes) else "ipc"
        error, handle = None, None
        try:
            self.native = self.C.Session(self.rank, self.world, layout.total, float(timeout), self.transport)
            handle = bytes(self.native.ipc_handle()) if (self.world > 1 and self.transport == "ipc") else b""
        except Exception as exc:  # tell the peers before raising, so nobody waits for a handle
            error = repr(exc)
        replies = control.all_gather_object((error, handle))
        errors = [f"rank {r}: {e}" for r, (e, _) in enumerate(replies) if e]
        if errors:
            if error is None:
                self.native.close()
            raise RuntimeError("workspace creation failed: " + "; ".join(errors))
        if self.world > 1:
            error = None
            try:
                if self.transport == "ipc":
                    self.native.open_peers([h for _, h in replies])
                else:
                    own = self.native.export_fd()
                    try:
                        fds = exchange_fds(control, own)
                    finally:
                        os.close(own)
                    self.native.open_peer_fds(fds)          # closes the descriptors
            except Exception as exc:  # a rank that cannot map a peer tells the others, so that all of them raise
                error = repr(exc)
            errors = [f"rank {r}: {e}" for r, e in enumerate(control.all_gather_object(error)) if e]
            if errors:
                shutdown_session(control, self.native)
                raise RuntimeError("mapping the peers' workspaces failed: " + "; ".join(errors))
        if not self.native.mapped():
            raise RuntimeError("a peer workspace is not mapped")
        self.stream = resolve_comm_stream(comm_stream, device)
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
        sync = (lambda: torch.cuda.synchronize(self.device)) if self.device.type == "cuda" else (lambda: None)
        sync()
        self.control.barrier()   # every rank's kernels are done: nothing writes into this workspace any more
        try:
            if not self.native.guard_intact():      # the canary zone behind the workspace (peers map it as well)
                warnings.warn("something wrote behind this rank's symmetric workspace; results of this buffer are suspect",
                              RuntimeWarning)
        except RuntimeError:
            pass
        try:
            shutdown_session(self.control, self.native, sync)
        finally:
            self.closed = True
            _busy_runtimes -= 1

    def __del__(self):
        if not getattr(self, "closed", True):
            warnings.warn("ElasticBuffer was never destroyed; call destroy() on every rank", ResourceWarning)


def runtime_busy() -> bool:
    return _busy_runtimes > 0
