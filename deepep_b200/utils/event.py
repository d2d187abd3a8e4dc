"""CUDA events and the overlap wrapper returned by every communication call.

Parity: ``deep_ep/utils/event.py:17-38`` (``EventHandle``) and ``:41-122``
(``EventOverlap``).  On a machine without CUDA the same classes work on a
no-op event so host-only tests exercise the ordering logic.
"""
from __future__ import annotations

from typing import Any, Callable, Optional, Tuple


def _cuda():
    import torch

    return torch.cuda if torch.cuda.is_available() else None


class _HostEvent:
    """Stand-in used when no CUDA device exists: host code is already ordered."""

    def record(self, stream=None):
        self.recorded = True

    def wait(self, stream=None):
        pass

    def synchronize(self):
        pass

    def query(self):
        return True


class EventHandle:
    """Records an event on ``stream`` (default: the current stream) at construction."""

    def __init__(self, stream: Any = None) -> None:
        cuda = _cuda()
        if cuda is None:
            self._device, self._stream, self._event = None, stream, _HostEvent()
            self._event.record(stream)
            return
        self._device = cuda.current_device()
        self._stream = cuda.current_stream(self._device) if stream is None else stream
        dev = getattr(getattr(self._stream, "device", None), "index", self._device)
        if dev is not None and dev != self._device:
            raise RuntimeError("Cannot record an event on another CUDA device")
        self._event = cuda.Event()
        self._event.record(self._stream)

    @property
    def event(self) -> Any:
        return self._event

    def current_stream_wait(self) -> None:
        cuda = _cuda()
        if cuda is None:
            return
        if cuda.current_device() != self._device:
            raise RuntimeError("Cannot wait for an event from another CUDA device")
        self._event.wait(cuda.current_stream(self._device))


class EventOverlap:
    """Completion event of an asynchronous call plus the tensors it keeps alive.

    An empty wrapper (``event is None``) is what synchronous calls return.
    """

    def __init__(self, event: Optional[EventHandle] = None, extra_tensors: Optional[Tuple[Any, ...]] = None) -> None:
        self.event = event
        self.extra_tensors = extra_tensors
        self.hook_after_wait: Optional[Callable] = None
        self._release_handle_by_call = False
        self._retained_objects = None
        self._stream_tensors: tuple = ()
        if isinstance(event, EventHandle) and extra_tensors is not None:
            self._track(extra_tensors)

    def _track(self, resources) -> None:
        import torch

        items = resources if isinstance(resources, (tuple, list)) else (resources,)
        flat = []
        for it in items:
            flat.extend(it if isinstance(it, (tuple, list)) else (it,))
        self._stream_tensors = tuple(t for t in flat if isinstance(t, torch.Tensor) and t.is_cuda)
        for t in self._stream_tensors:  # the producer stream used them
            t.record_stream(self.event._stream)

    @classmethod
    def _from_resources(cls, event: EventHandle, resources: Tuple[Any, ...]) -> "EventOverlap":
        out = cls(event)
        out._retained_objects = resources
        out._track(resources)
        return out

    def current_stream_wait(self, release_handle: bool = False) -> Any:
        """Make the current stream wait for the call.  On the empty wrapper of a synchronous call there is nothing left
        to wait for (the current stream was already ordered after the call), so callers may use one code path for both
        forms, as the usage examples of the reference do (``README.md:168-196``)."""
        if self.event is not None:
            self.event.current_stream_wait()
        cuda = _cuda()
        if self.event is not None and cuda is not None and self._stream_tensors:
            cur = cuda.current_stream(self.event._device)
            for t in self._stream_tensors:  # the consumer stream uses them from now on
                t.record_stream(cur)
        result = None
        if self.hook_after_wait is not None:
            hook, self.hook_after_wait = self.hook_after_wait, None
            result = hook()
        if release_handle:
            self.event, self._retained_objects, self._stream_tensors = None, None, ()
        return result

    def wait(self) -> Any:
        return self.current_stream_wait()

    def register_hook_after_wait(self, hook_after_wait: Callable) -> None:
        assert self.hook_after_wait is None, "A hook is already registered on this `EventOverlap`"
        self.hook_after_wait = hook_after_wait

    def __call__(self, release_handle: bool = False) -> "EventOverlap":
        self._release_handle_by_call = release_handle
        return self

    def __enter__(self) -> Any:
        return self

    def __exit__(self, exc_type, exc_val, exc_tb) -> None:
        if self.event is not None:
            self.current_stream_wait(release_handle=self._release_handle_by_call)
        self._release_handle_by_call = False


__all__ = ["EventHandle", "EventOverlap"]
