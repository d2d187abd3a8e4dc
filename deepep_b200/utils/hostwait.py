"""Bounded host-side wait for work queued on a CUDA stream.

A fresh dispatch reads the row counts back on the host, so the host has to wait for the routing kernel.  The kernels
bound their own waits and return, so this wait normally ends by itself; the limit here covers what the kernels cannot
see (a device that stopped making progress at all).  Parity: the reference's host wait on its pinned mailbox, which
raises ``[DEEPEP_CPU_TIMEOUT]`` after ``DEEPEP_CPU_TIMEOUT_SECONDS``
(``csrc/direct/runtime/shmem_instance.cpp:677-693`` of the reference).
"""
from __future__ import annotations

import os
import time


class HostTimeout(RuntimeError):
    pass


def cpu_timeout_seconds(default: float) -> float:
    """Host wait limit: ``DEEPEP_CPU_TIMEOUT_SECONDS`` overrides the constructor's ``num_cpu_timeout_secs``."""
    if "DEEPEP_CPU_TIMEOUT_SECONDS" in os.environ:
        value = float(os.environ["DEEPEP_CPU_TIMEOUT_SECONDS"])
        if not 1 <= value <= 3600:
            raise ValueError("DEEPEP_CPU_TIMEOUT_SECONDS must be in [1, 3600] seconds")
        return value
    return float(default)


def wait_for_event(event, timeout_seconds: float, what: str, spin_seconds: float = 0.005, clock=time.monotonic,
                   sleep=time.sleep) -> float:
    """Poll ``event.query()`` until it reports completion; returns the seconds waited.  The first ``spin_seconds`` are
    polled without pause (the kernels waited for take tens of microseconds), after that the thread sleeps 0.2 ms between
    polls.  Raises :class:`HostTimeout` when ``timeout_seconds`` pass first; the work is then still queued, and the
    caller must treat the buffer as failed."""
    start = clock()
    while not event.query():
        waited = clock() - start
        if waited > timeout_seconds:
            raise HostTimeout(f"[DEEPEP_CPU_TIMEOUT] {what} did not finish within {timeout_seconds:.0f} s on the device")
        if waited > spin_seconds:
            sleep(0.0002)
    return clock() - start


__all__ = ["HostTimeout", "cpu_timeout_seconds", "wait_for_event"]
