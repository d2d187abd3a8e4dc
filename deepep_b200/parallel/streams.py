"""One communication stream per process and GPU, for callers that want every buffer's traffic on a single timeline.

An :class:`~deepep_b200.parallel.elastic.ElasticBuffer` normally owns a stream of its own, so a prefill buffer and a
decode buffer overlap.  Serving stacks written for upstream DeepEP sometimes rely on the opposite: all buffers of a
process share one stream, and ordering work after that one stream orders it after every buffer.
``get_global_comm_stream`` returns that stream (parity: the function of the same name in the reference,
``deep_ep/backends/direct/buffer.py:1362-1383``; its V1 and V2 buffers share it); pass ``comm_stream="global"`` to a
buffer to make it use it.

The registry is keyed by ``(process id, device index)``: a forked child never inherits a parent's stream object, and
each GPU of a multi-GPU process gets its own.  Creation happens under a lock, and a failed creation leaves no entry.
"""
from __future__ import annotations

import os
import threading
from typing import Any, Dict, Optional, Tuple

import torch

_streams: Dict[Tuple[int, int], Any] = {}
_lock = threading.Lock()


def get_global_comm_stream(device: Optional[int] = None) -> Any:
    """The shared communication stream of this process on ``device`` (default: the current device)."""
    index = torch.cuda.current_device() if device is None else int(getattr(device, "index", device))
    key = (os.getpid(), index)
    with _lock:
        found = _streams.get(key)
        if found is None:
            found = torch.cuda.Stream(device=index)          # raises before anything is stored
            _streams[key] = found
        return found


def resolve_comm_stream(choice: Any, device: torch.device) -> Any:
    """Stream for a new buffer on ``device``: ``None`` makes a private one, ``"global"`` takes the shared one, a stream
    object is used as given (it must live on ``device``).  On a machine without CUDA there is no stream at all."""
    if device.type != "cuda":
        if choice not in (None, "global"):
            raise ValueError("a communication stream needs a CUDA device")
        return None
    if choice is None:
        return torch.cuda.Stream(device=device)
    if isinstance(choice, str):
        if choice != "global":
            raise ValueError("comm_stream must be None, 'global' or a CUDA stream")
        return get_global_comm_stream(device.index)
    where = getattr(getattr(choice, "device", None), "index", None)
    if where is not None and device.index is not None and where != device.index:
        raise ValueError(f"comm_stream lives on GPU {where}, the buffer on GPU {device.index}")
    return choice


__all__ = ["get_global_comm_stream", "resolve_comm_stream"]
