"""The bounded host-side wait (``deepep_b200/utils/hostwait.py``) with stand-in events and clocks: it returns when the
event completes, sleeps only after the spin phase, and raises ``[DEEPEP_CPU_TIMEOUT]`` when the limit passes first
(the failure is a stand-in event that never completes; no device is involved)."""
import pytest

from deepep_b200.utils import hostwait as HW


class Event:
    def __init__(self, polls_until_done):
        self.left = polls_until_done

    def query(self):
        self.left -= 1
        return self.left < 0


class Clock:
    """Every reading advances the time by ``step`` seconds."""
    def __init__(self, step):
        self.now, self.step, self.sleeps = 0.0, step, []

    def __call__(self):
        self.now += self.step
        return self.now

    def sleep(self, seconds):
        self.sleeps.append(seconds)
        self.now += seconds


def test_returns_when_the_event_completes():
    clock = Clock(0.001)
    waited = HW.wait_for_event(Event(3), 10.0, "x", clock=clock, sleep=clock.sleep)
    assert clock.sleeps == [] and 0 < waited < 0.01              # done within the spin phase: no sleep at all
    assert HW.wait_for_event(Event(0), 10.0, "x", clock=clock, sleep=clock.sleep) >= 0


def test_sleeps_between_polls_after_the_spin_phase():
    clock = Clock(0.002)
    HW.wait_for_event(Event(10), 10.0, "x", spin_seconds=0.005, clock=clock, sleep=clock.sleep)
    assert clock.sleeps and all(s == 0.0002 for s in clock.sleeps) and len(clock.sleeps) < 10


def test_gives_up_after_the_limit():
    clock = Clock(0.5)
    with pytest.raises(HW.HostTimeout, match=r"\[DEEPEP_CPU_TIMEOUT\] the routing layout pass did not finish within 2 s"):
        HW.wait_for_event(Event(10 ** 9), 2.0, "the routing layout pass", clock=clock, sleep=clock.sleep)
    assert clock.now < 10


def test_environment_overrides_the_constructor(monkeypatch):
    monkeypatch.delenv("DEEPEP_CPU_TIMEOUT_SECONDS", raising=False)
    assert HW.cpu_timeout_seconds(300) == 300.0
    monkeypatch.setenv("DEEPEP_CPU_TIMEOUT_SECONDS", "45")
    assert HW.cpu_timeout_seconds(300) == 45.0
    monkeypatch.setenv("DEEPEP_CPU_TIMEOUT_SECONDS", "0")
    with pytest.raises(ValueError, match="3600"):
        HW.cpu_timeout_seconds(300)


def test_the_engine_turns_a_host_timeout_into_a_communication_error(monkeypatch):
    """``CudaEngine._host_wait`` with stand-ins for the stream and the event: it records an event on the stream it was
    given, polls it, synchronises the stream at the end, and raises ``CommunicationError`` when the limit passes."""
    import types

    import torch

    from deepep_b200.parallel import engine_cuda as EC

    log = []

    class FakeEvent:
        polls_until_done = 2

        def record(self, stream):
            log.append(("record", stream.name))
            self.left = self.polls_until_done

        def query(self):
            self.left -= 1
            return self.left < 0

    class FakeStream:
        name = "comm"

        def synchronize(self):
            log.append(("synchronize", self.name))

    monkeypatch.setattr(torch.cuda, "Event", FakeEvent)
    engine = types.SimpleNamespace(device=torch.device("cpu"), host_timeout=5.0)
    EC.CudaEngine._host_wait(engine, FakeStream(), "the routing layout pass")
    assert log == [("record", "comm"), ("synchronize", "comm")]
    FakeEvent.polls_until_done = 10 ** 9
    engine.host_timeout = 0.05
    with pytest.raises(EC.CommunicationError, match=r"\[DEEPEP_CPU_TIMEOUT\] the routing layout pass .* restart the distributed job"):
        EC.CudaEngine._host_wait(engine, FakeStream(), "the routing layout pass")
