"""The stream / event contract of ``ElasticBuffer`` with recording stand-ins for the streams (no GPU): which stream waits
for what, in which order, in the synchronous and the asynchronous form, with and without ``previous_event``.

Parity: the reference checks the same ordering with fake events and a fake native module
(``tests/runtime/test_runtime.py``, ``tests/runtime/test_communication_stream.py``).  The data path underneath is the
CPU engine, so results are still compared with the oracle's round-trip answer.
"""
import contextlib

import pytest
import torch

import deepep_b200 as deep_ep
from deepep_b200.oracle import reference as R
from helpers import make_routes, make_weights


class FakeStream:
    def __init__(self, name, log):
        self.name, self.log = name, log

    def wait_event(self, event):
        self.log.append((self.name, "wait_event", event))

    def wait_stream(self, other):
        self.log.append((self.name, "wait_stream", other.name))

    def synchronize(self):
        self.log.append((self.name, "synchronize"))


class FakeRuntime:
    def __init__(self, log):
        self.stream, self.failed, self.closed = FakeStream("comm", log), False, False

    def ensure_alive(self):
        if self.closed:
            raise RuntimeError("the buffer was destroyed")

    def close(self):
        self.closed = True


@pytest.fixture
def wired(monkeypatch):
    """A CPU-engine buffer whose runtime and current stream are recording stand-ins."""
    if torch.cuda.is_available():
        pytest.skip("the stand-ins replace torch.cuda.current_stream; CPU-engine test")
    log = []
    buf = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=64, hidden=128, num_topk=3, explicitly_destroy=True, device="cpu")
    buf.runtime = FakeRuntime(log)
    cur = FakeStream("cur", log)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda device=None: cur)
    contexts = []

    def on(comm):                    # what `with torch.cuda.stream(comm)` would do: remember which stream allocations use
        contexts.append(None if comm is None else comm.name)
        return contextlib.nullcontext()

    monkeypatch.setattr(buf, "_on", on)
    T, E = 40, 8
    x = torch.randn(T, 128).bfloat16()
    idx, w = make_routes("invalid", T, E, 3, 1, 5), make_weights(T, 3, 2)
    yield buf, log, contexts, (x, idx, w, E)
    buf.destroy()
    assert buf.runtime.closed


def test_synchronous_call_orders_both_ways(wired):
    buf, log, contexts, (x, idx, w, E) = wired
    rx, _, rw, handle, event = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True)
    # the communication stream starts after the current stream's work; the current stream continues after the call
    assert log == [("comm", "wait_stream", "cur"), ("cur", "wait_stream", "comm")]
    assert event.event is None and contexts[0] is None               # outputs from the current stream's pool
    del log[:]
    out, _, event = buf.combine((rx.float() * rw[:, None]).bfloat16(), handle)
    assert log == [("comm", "wait_stream", "cur"), ("cur", "wait_stream", "comm")] and event.event is None
    want = R.expected_roundtrip([x], [idx], [w], E)[0]
    assert torch.allclose(out.float(), want, rtol=0.02, atol=0.02)


def test_previous_event_replaces_the_wait_for_the_current_stream(wired):
    buf, log, contexts, (x, idx, w, E) = wired
    first, second = deep_ep.EventHandle(), deep_ep.EventOverlap(deep_ep.EventHandle())
    rx, _, _, handle, event = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True,
                                           previous_event=first, previous_event_before_epilogue=second)
    assert log == [("comm", "wait_event", first.event), ("comm", "wait_event", second.event.event), ("cur", "wait_stream", "comm")]
    assert contexts[0] == "comm"       # ordered after an event: outputs come from the communication stream's pool
    del log[:], contexts[:]
    buf.dispatch(x, handle=handle, previous_event=first)
    assert log == [("comm", "wait_event", first.event), ("cur", "wait_stream", "comm")] and contexts == ["comm"]
    del log[:], contexts[:]
    buf.combine(rx, handle, previous_event=second)
    assert log == [("comm", "wait_event", second.event.event), ("cur", "wait_stream", "comm")] and contexts == ["comm"]


def test_asynchronous_call_returns_an_event_that_keeps_the_tensors(wired):
    buf, log, contexts, (x, idx, w, E) = wired
    rx, _, rw, handle, event = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True,
                                            async_with_compute_stream=True, allocate_on_comm_stream=True)
    assert log == [("comm", "wait_stream", "cur")]                    # the current stream does not wait by itself
    assert contexts[0] == "comm" and event.event is not None and event.event._stream is buf.runtime.stream
    kept = [t for t in event._retained_objects if isinstance(t, torch.Tensor)]
    assert any(t is rx for t in kept) and any(t is x for t in kept) and any(t is idx for t in kept)
    ran = []
    event.register_hook_after_wait(lambda: ran.append(True))
    with event(release_handle=True):
        pass
    assert ran == [True] and event.event is None and event._retained_objects is None
    del log[:]
    out, _, done = buf.combine(rx, handle, async_with_compute_stream=True)
    assert log == [("comm", "wait_stream", "cur")] and done.event is not None
    done.current_stream_wait()


def test_barrier_and_stream_getters(wired):
    buf, log, _, _ = wired
    assert buf.get_comm_stream() is buf.runtime.stream
    assert isinstance(buf.capture(), deep_ep.EventHandle)
    buf.barrier()
    assert log == [("comm", "wait_stream", "cur"), ("cur", "wait_stream", "comm")]
    del log[:]
    buf.barrier(use_comm_stream=False, with_cpu_sync=True)              # on the current stream, then a host wait
    assert log == [("cur", "synchronize")]
    buf.runtime.closed = True
    with pytest.raises(RuntimeError, match="destroyed"):
        buf.get_comm_stream()
    buf.runtime.closed = False
