"""Several expert-parallel ranks emulated on ONE GPU inside single cooperative launches.

Every virtual rank owns a real workspace and a real :class:`Session`; the
"peer mappings" are simply the other workspaces' addresses on the same
device.  Kernels pick their rank from ``blockIdx.y`` and run exactly the code
a multi-GPU job runs, including all release/acquire flag traffic, so the
protocol can be validated against the CPU oracle without a second GPU.
(Ranks that wait on one another must never be separate launches on one GPU;
one cooperative launch guarantees that all of them are resident.)
"""
from __future__ import annotations

import torch

from ..ops import require_native
from .engine_cuda import CudaEngine


class VirtualWorld:
    def __init__(self, world: int, num_max_tokens_per_rank: int, hidden: int, num_topk: int, device=None,
                 timeout: float = 20.0, num_sms: int = 0, ll_bytes: int = 0, mega_bytes: int = 0, partial_tokens: int = 0):
        C = require_native("VirtualWorld")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        torch.cuda.set_device(self.device)
        self.layout = C.make_layout(world, num_max_tokens_per_rank, hidden, num_topk, ll_bytes, mega_bytes, partial_tokens)
        self.sessions = [C.Session(r, world, self.layout.total, timeout) for r in range(world)]
        bases = [s.workspace for s in self.sessions]
        for s in self.sessions:
            s.attach_peers(bases)
        self.engine = CudaEngine(self.sessions, self.layout, self.device, num_sms=num_sms)
        self.world = world

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        # every workspace ends in a canary zone: a kernel that wrote past a workspace is reported here
        damaged = [i for i, s in enumerate(self.sessions) if not s.closed and not s.guard_intact()]
        for s in self.sessions:
            s.close()
        if damaged:
            raise RuntimeError(f"something wrote behind the workspace of virtual rank(s) {damaged}")

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
