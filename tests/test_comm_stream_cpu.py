"""The process-wide communication stream: one per process and device, made once under concurrent first use, never
published when its creation fails; and the ``comm_stream`` choice of a buffer.  The CUDA stream class is replaced by a
recording stand-in, so no device is needed.  Parity: the reference's shared-stream tests
(``tests/runtime/test_communication_stream.py``)."""
import threading
from concurrent.futures import ThreadPoolExecutor

import pytest
import torch

from deepep_b200.parallel import streams as S


class _FakeCuda:
    def __init__(self):
        self.made, self.current, self.fail = [], 0, False

    def stream(self, device=None):
        if self.fail:
            raise RuntimeError("no stream today")
        index = getattr(device, "index", device)
        made = type("FakeStream", (), {"device": torch.device("cuda", index)})()
        self.made.append(made)
        return made


@pytest.fixture
def cuda(monkeypatch):
    fake = _FakeCuda()
    monkeypatch.setattr(torch.cuda, "Stream", fake.stream)
    monkeypatch.setattr(torch.cuda, "current_device", lambda: fake.current)
    monkeypatch.setattr(S, "_streams", {})
    return fake


def test_one_stream_per_process_and_device(cuda, monkeypatch):
    import deepep_b200.buffer as v1
    import deepep_b200.parallel.elastic as v2

    first = v1.get_global_comm_stream()
    assert v2.get_global_comm_stream() is first and S.get_global_comm_stream(0) is first
    cuda.current = 1
    other = v2.get_global_comm_stream()
    assert other is not first and other.device.index == 1
    assert S.get_global_comm_stream(torch.device("cuda", 0)) is first
    pid = S.os.getpid()
    monkeypatch.setattr(S.os, "getpid", lambda: pid + 1)           # what a forked child sees
    assert S.get_global_comm_stream(0) is not first and len(cuda.made) == 3


def test_concurrent_first_use_makes_one_stream(cuda):
    gate = threading.Barrier(8)

    def grab(_):
        gate.wait(timeout=10)
        return S.get_global_comm_stream()

    with ThreadPoolExecutor(max_workers=8) as pool:
        got = list(pool.map(grab, range(8)))
    assert len(cuda.made) == 1 and all(g is got[0] for g in got)


def test_failed_creation_leaves_no_entry(cuda):
    cuda.fail = True
    with pytest.raises(RuntimeError, match="no stream today"):
        S.get_global_comm_stream()
    assert S._streams == {}
    cuda.fail = False
    assert S.get_global_comm_stream() is S.get_global_comm_stream() and len(cuda.made) == 1


def test_buffer_stream_choices(cuda):
    dev = torch.device("cuda", 0)
    own_a, own_b = S.resolve_comm_stream(None, dev), S.resolve_comm_stream(None, dev)
    assert own_a is not own_b
    shared = S.resolve_comm_stream("global", dev)
    assert shared is S.get_global_comm_stream(0) and S.resolve_comm_stream("global", dev) is shared
    assert S.resolve_comm_stream(own_a, dev) is own_a
    with pytest.raises(ValueError, match="lives on GPU 0"):
        S.resolve_comm_stream(own_a, torch.device("cuda", 1))
    with pytest.raises(ValueError):
        S.resolve_comm_stream("shared", dev)
    assert S.resolve_comm_stream("global", torch.device("cpu")) is None and S.resolve_comm_stream(None, torch.device("cpu")) is None
    with pytest.raises(ValueError, match="needs a CUDA device"):
        S.resolve_comm_stream(own_a, torch.device("cpu"))


def test_constructor_refuses_an_unknown_choice():
    import deepep_b200 as deep_ep

    with pytest.raises(ValueError, match="comm_stream"):
        deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=8, hidden=64, num_topk=2, comm_stream="mine", device="cpu")
    buf = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=8, hidden=64, num_topk=2, comm_stream="global", device="cpu",
                                explicitly_destroy=True)
    assert buf.get_comm_stream() is None            # the CPU engine has no streams
    buf.destroy()
