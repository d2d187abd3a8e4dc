"""CUDA events and the completion object that every communication call returns.

Two public classes with the names and methods of upstream DeepEP (parity: ``deep_ep/utils/event.py`` of the
reference, ``EventHandle`` and ``EventOverlap``):

* :class:`EventHandle` is one ``torch.cuda.Event`` recorded at construction, with the stream and device it was
  recorded on.  Besides the upstream ``current_stream_wait`` it offers ``query`` and ``synchronize`` so host code
  can poll it with a deadline.
* :class:`EventOverlap` pairs such an event with what must outlive it.  The caching allocator hands a block back
  as soon as the last Python reference dies *on the allocating stream's timeline*; a tensor produced on the
  communication stream and consumed on the compute stream therefore has to be announced to both
  (``Tensor.record_stream``).  That bookkeeping lives in :class:`_Lease`.

Without a CUDA device both classes still work: the event is a host stand-in that is always complete, which lets
the ordering logic of the callers run in CPU tests.
"""
from __future__ import annotations

from typing import Any, Callable, Iterable, Optional, Tuple

import torch


class _CompletedEvent:
    """Host stand-in for a device event: everything before it has already happened."""

    def record(self, stream: Any = None) -> None:
        self.recorded = True

    def wait(self, stream: Any = None) -> None:
        return None

    def synchronize(self) -> None:
        return None

    def query(self) -> bool:
        return True


def _device_index_of(stream: Any, fallback: Optional[int]) -> Optional[int]:
    device = getattr(stream, "device", None)
    return getattr(device, "index", fallback) if device is not None else fallback


class EventHandle:
    """An event recorded on ``stream`` (the current stream when omitted) the moment the object is made."""

    def __init__(self, stream: Any = None) -> None:
        if not torch.cuda.is_available():
            self._device, self._stream, self._event = None, stream, _CompletedEvent()
        else:
            self._device = torch.cuda.current_device()
            self._stream = stream if stream is not None else torch.cuda.current_stream(self._device)
            if _device_index_of(self._stream, self._device) != self._device:
                raise RuntimeError("Cannot record an event on another CUDA device")
            self._event = torch.cuda.Event()
        self._event.record(self._stream)

    event = property(lambda self: self._event, doc="The framework event underneath.")
    stream = property(lambda self: self._stream, doc="The stream the event was recorded on.")
    device = property(lambda self: self._device, doc="Index of the device, ``None`` on a machine without CUDA.")

    def query(self) -> bool:
        """Whether the work before the event has finished (never blocks)."""
        return bool(self._event.query())

    def synchronize(self) -> None:
        """Block the host until the work before the event has finished."""
        self._event.synchronize()

    def current_stream_wait(self) -> None:
        """Order the current stream after the event (device-side wait; the host does not block)."""
        if self._device is None:
            return
        if torch.cuda.current_device() != self._device:
            raise RuntimeError("Cannot wait for an event from another CUDA device")
        self._event.wait(torch.cuda.current_stream(self._device))


class _Lease:
    """What an asynchronous call keeps alive, and the device tensors among it whose streams must be announced."""

    __slots__ = ("owned", "tensors")

    def __init__(self) -> None:
        self.owned: Any = None
        self.tensors: Tuple[torch.Tensor, ...] = ()

    @staticmethod
    def _walk(item: Any) -> Iterable[Any]:
        if isinstance(item, (tuple, list)):
            for inner in item:
                yield from _Lease._walk(inner)
        else:
            yield item

    def adopt(self, resources: Any, producer: Any) -> None:
        self.tensors = tuple(t for t in self._walk(resources) if isinstance(t, torch.Tensor) and t.is_cuda)
        self.announce(producer)                           # holds even if the wrapper is dropped without a wait

    def announce(self, stream: Any) -> None:
        for tensor in self.tensors:
            tensor.record_stream(stream)

    def release(self) -> None:
        self.owned, self.tensors = None, ()


class EventOverlap:
    """Completion of one communication call.

    ``event`` is ``None`` for a synchronous call (the current stream was already ordered after it); waiting on such
    an object does nothing, so one code path serves both forms, as in the usage examples of the reference
    (``README.md:168-196``).  ``extra_tensors`` is kept until the object itself goes away, like upstream.  A hook
    registered with :meth:`register_hook_after_wait` runs once, right after the wait is enqueued, and its result is
    what the wait returns.  As a context manager the wait happens on leaving the block; calling the object first
    (``with ev(release_handle=True):``) also drops the event and everything leased at that point.
    """

    def __init__(self, event: Optional[EventHandle] = None, extra_tensors: Optional[Tuple[Any, ...]] = None) -> None:
        self.event = event
        self.extra_tensors = extra_tensors
        self.hook_after_wait: Optional[Callable[[], Any]] = None
        self._lease = _Lease()
        self._release_on_exit = False
        if extra_tensors is not None and isinstance(event, EventHandle):
            self._lease.adopt(extra_tensors, event.stream)

    @classmethod
    def _from_resources(cls, event: EventHandle, resources: Tuple[Any, ...]) -> "EventOverlap":
        """Completion object that owns ``resources`` (handles, staging tensors) without exposing them as ``extra_tensors``."""
        made = cls(event)
        made._lease.owned = resources
        made._lease.adopt(resources, event.stream)
        return made

    @property
    def _retained_objects(self) -> Any:
        return self._lease.owned

    def current_stream_wait(self, release_handle: bool = False) -> Any:
        handle = self.event
        if handle is not None:
            handle.current_stream_wait()
            device = getattr(handle, "device", None)                   # a duck-typed event carries no lease
            if device is not None and self._lease.tensors:             # the consumer stream uses them from now on
                self._lease.announce(torch.cuda.current_stream(device))
        outcome = None
        if self.hook_after_wait is not None:
            outcome = self.hook_after_wait()                           # a hook that raises stays registered for a retry
            self.hook_after_wait = None
        if release_handle:
            self.event = None
            self._lease.release()
        return outcome

    def wait(self) -> Any:
        """Same as :meth:`current_stream_wait`; returns the hook's result."""
        return self.current_stream_wait()

    def register_hook_after_wait(self, hook_after_wait: Callable[[], Any]) -> None:
        assert self.hook_after_wait is None, "A hook is already registered on this `EventOverlap`"
        self.hook_after_wait = hook_after_wait

    def __call__(self, release_handle: bool = False) -> "EventOverlap":
        self._release_on_exit = bool(release_handle)
        return self

    def __enter__(self) -> "EventOverlap":
        return self

    def __exit__(self, exc_type: Any, exc_val: Any, exc_tb: Any) -> None:
        release, self._release_on_exit = self._release_on_exit, False
        if self.event is not None:
            self.current_stream_wait(release_handle=release)


__all__ = ["EventHandle", "EventOverlap"]
