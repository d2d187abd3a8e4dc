"""Machine detection, cross-rank consensus and the peer-access preflight that run when a buffer is constructed.

The reference selects a backend from the machine it finds (``deep_ep/backends/__init__.py`` with ``machine_type``
``"auto"``), lets the ranks agree on it and refuses a job whose ranks see different machines.  Here there is one data
plane (a symmetric workspace that all GPUs of one NVLink / NVSwitch domain map), so detection answers three questions
before any memory is shared: is every rank on the same kind of GPU, does every rank own a different GPU of the same
host, and can every GPU reach every other one by peer access.  A job that fails one of them gets one clear error on
every rank instead of a mapping failure or a hang later.
"""
from __future__ import annotations

import os
import socket
from dataclasses import asdict, dataclass
from typing import Dict, Optional, Sequence

import torch

KINDS = ("nvswitch", "single", "cpu")


@dataclass
class RankMachine:
    """What one rank sees."""
    rank: int
    host: str                       # ranks of one buffer share a host (one NVLink domain)
    kind: str                       # "cpu" without a GPU, else "single" (one visible GPU) or "nvswitch"
    device: int = -1                # CUDA device index of this rank
    uuid: str = ""                  # stable identity of the GPU (two ranks must not share one)
    name: str = ""
    capability: Sequence[int] = (0, 0)
    sm_count: int = 0
    visible: int = 0                # GPUs visible to the process
    peer_access: Optional[Dict[int, bool]] = None   # device index -> reachable by peer access from this rank's GPU


def detect(rank: int, device: Optional[torch.device] = None) -> RankMachine:
    """Describe this rank's machine.  Read-only: nothing is enabled or changed."""
    host = os.environ.get("DEEPEP_HOST_ID") or socket.gethostname()
    if device is None or torch.device(device).type != "cuda" or not torch.cuda.is_available():
        return RankMachine(rank=rank, host=host, kind="cpu")
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    props = torch.cuda.get_device_properties(index)
    visible = torch.cuda.device_count()
    access = {d: (d == index or bool(torch.cuda.can_device_access_peer(index, d))) for d in range(visible)}
    return RankMachine(rank=rank, host=host, kind="single" if visible == 1 else "nvswitch", device=index,
                       uuid=str(getattr(props, "uuid", "")), name=props.name, capability=(props.major, props.minor),
                       sm_count=props.multi_processor_count, visible=visible, peer_access=access)


def check_consensus(machines: Sequence[RankMachine], machine_type: Optional[str] = "auto") -> str:
    """Validate what all ranks reported; returns the agreed machine kind or raises ``RuntimeError`` naming the ranks.

    Rules: all ranks on CPU or all on GPUs; one host; the same GPU model and compute capability everywhere; compute
    capability 10.x (the kernels are built for sm_100a only); no GPU used by two ranks; every rank's GPU reaches the
    GPU of every other rank by peer access.  ``machine_type`` other than ``"auto"`` must match what was found.
    """
    if not machines:
        raise RuntimeError("no rank reported its machine")
    world = len(machines)
    kinds = {m.kind == "cpu" for m in machines}
    if len(kinds) > 1:
        raise RuntimeError("some ranks run on GPUs and some on the CPU: "
                           + ", ".join(f"rank {m.rank}: {m.kind}" for m in machines))
    if machines[0].kind == "cpu":
        kind = "cpu"
    else:
        hosts = sorted({m.host for m in machines})
        if len(hosts) > 1:
            raise RuntimeError(f"the ranks of one buffer must share one NVLink domain (one host); found hosts {hosts}")
        models = sorted({(m.name, tuple(m.capability)) for m in machines})
        if len(models) > 1:
            raise RuntimeError(f"ranks see different GPUs: {models}")
        major = tuple(machines[0].capability)[0]
        if major != 10:
            raise RuntimeError(f"the kernels are built for compute capability 10.x (B200); found {machines[0].name} "
                               f"with {tuple(machines[0].capability)}")
        owners: Dict[str, int] = {}
        for m in machines:
            key = m.uuid or f"device{m.device}"
            if key in owners and world > 1:
                raise RuntimeError(f"ranks {owners[key]} and {m.rank} use the same GPU ({key}); one GPU per rank is required")
            owners[key] = m.rank
        blocked = []
        for m in machines:
            for peer in machines:
                if peer.rank != m.rank and not (m.peer_access or {}).get(peer.device, False):
                    blocked.append((m.rank, peer.rank))
        if blocked:
            raise RuntimeError(f"no peer access between the GPUs of these (rank, peer rank) pairs: {blocked}; "
                               "all GPUs of a buffer must be in one NVLink / NVSwitch domain")
        kind = "single" if world == 1 else "nvswitch"
    if machine_type not in (None, "auto"):
        wanted = "nvswitch" if machine_type in ("nvswitch", "b200") else machine_type
        if wanted not in KINDS:
            raise ValueError(f"machine_type must be 'auto' or one of {KINDS}")
        if wanted != kind and not (wanted == "nvswitch" and kind == "single"):
            raise RuntimeError(f"machine_type={machine_type!r} was requested but the ranks found a {kind!r} machine")
    return kind


def agree(control, device: Optional[torch.device], machine_type: Optional[str] = "auto", details: bool = False):
    """Collective: every rank detects its machine, all ranks exchange the findings and apply the same rules, so all of
    them return the same kind or raise the same error.  ``details=True`` returns ``(kind, selection)`` where
    ``selection`` records what was asked for, what was found and every rank's report (the reference's
    ``buffer.machine_selection``)."""
    mine = detect(control.rank, device)
    gathered = control.all_gather_object(asdict(mine))
    reports = [RankMachine(**r) for r in gathered]
    kind = check_consensus(reports, machine_type)
    if not details:
        return kind
    return kind, {"machine_type": kind, "requested": machine_type or "auto", "source": "detected and agreed by all ranks",
                  "ranks": [dict(r) for r in gathered]}


def main(argv: Optional[Sequence[str]] = None) -> int:
    """``python -m deepep_b200.parallel.topology [--ranks N]``: print what this process sees, as JSON, and whether N
    ranks (default: one per visible GPU) on this machine would pass the constructor's check.  Read-only.
    Parity: the reference's machine probe (``scripts/check_machine.py``)."""
    import argparse
    import json

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--ranks", type=int, default=0, help="ranks of the planned job (0: one per visible GPU)")
    args = ap.parse_args(argv)
    gpus = torch.cuda.device_count() if torch.cuda.is_available() else 0
    ranks = args.ranks or max(gpus, 1)
    if gpus:
        reports = [detect(r, torch.device("cuda", r % gpus)) for r in range(ranks)]
    else:
        reports = [detect(r, None) for r in range(ranks)]
    out = {"host": reports[0].host, "visible_gpus": gpus, "ranks": ranks, "reports": [asdict(m) for m in reports]}
    try:
        out["machine_type"], out["ok"] = check_consensus(reports), True
    except RuntimeError as exc:
        out["machine_type"], out["ok"], out["error"] = None, False, str(exc)
    print(json.dumps(out, indent=1, default=list))
    return 0 if out["ok"] else 1


__all__ = ["KINDS", "RankMachine", "agree", "check_consensus", "detect", "main"]


if __name__ == "__main__":
    raise SystemExit(main())
