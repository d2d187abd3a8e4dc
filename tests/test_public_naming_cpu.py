"""Upstream spellings and platform-neutral spellings name the same parameters: either may be used, both together only
with equal values, and neither changes a default.  Parity: ``tests/api/test_public_naming.py`` of the reference."""
import inspect

import pytest

import deepep_b200 as deep_ep
from deepep_b200 import _compat


def test_alias_wrapper_rules():
    def implementation(x, num_sms=32, *, previous_event=None, async_finish=False):
        return x, num_sms, previous_event, async_finish

    call = _compat.keyword_aliases(implementation, {"num_compute_units": "num_sms", "num_aiv": "num_sms"})
    x, event = object(), object()
    assert call(x) == (x, 32, None, False)
    for keyword in ("num_sms", "num_compute_units", "num_aiv"):
        assert call(x, **{keyword: 64}, previous_event=event, async_finish=True) == (x, 64, event, True)
    assert call(x, 64, num_aiv=64)[1] == 64 and call(x, num_sms=64, num_compute_units=64, num_aiv=64)[1] == 64
    for kwargs in ({"num_aiv": 32}, {"num_compute_units": 32}):
        with pytest.raises(TypeError, match="conflicting"):
            call(x, 64, **kwargs)
    with pytest.raises(TypeError, match="conflicting"):
        call(x, num_compute_units=32, num_sms=64)
    with pytest.raises(TypeError, match="unexpected"):
        call(x, unknown=1)
    with pytest.raises(ValueError, match="unknown implementation parameter"):
        _compat.public_keywords(lambda compute_read_gbs=200: None, {"sm_read_gbs": "compute_unit_read_gbs"})
    shown = _compat.public_keywords(implementation, {"num_compute_units": "num_sms"})
    assert list(inspect.signature(shown).parameters) == ["x", "num_compute_units", "previous_event", "async_finish"]


def test_config_and_handle_spellings():
    upstream, platform, ascend = deep_ep.Config(num_sms=32), deep_ep.Config(num_compute_units=32), deep_ep.Config(num_aiv=32)
    assert upstream.num_sms == platform.num_sms == ascend.num_sms == 32 == platform.num_compute_units == ascend.num_aiv
    assert upstream.get_nvl_buffer_size_hint(14336, 8, 129) == platform.get_scaleup_buffer_size_hint(14336, 8, 129)
    assert upstream.get_rdma_buffer_size_hint(14336, 8) == platform.get_scaleout_buffer_size_hint(14336, 8) == 0
    both = deep_ep.Config(32, num_max_scaleup_chunked_send_tokens=8, num_max_shmem_chunked_recv_tokens=128)
    assert (both.num_max_nvl_chunked_send_tokens, both.num_max_nvl_chunked_recv_tokens) == (8, 128)
    with pytest.raises(TypeError, match="conflicting"):
        deep_ep.Config(32, num_compute_units=64)
    platform.num_compute_units = 48
    assert platform.num_sms == 48
    handle = object.__new__(deep_ep.EPHandle)
    handle.num_sms = 32
    assert handle.num_compute_units == 32
    handle.num_compute_units = 64
    assert handle.num_sms == 64


def test_buffer_spellings(monkeypatch):
    old = deep_ep.Buffer.num_sms
    try:
        deep_ep.Buffer.set_num_sms(new_num_compute_units=26)
        assert deep_ep.Buffer.num_sms == 26
        deep_ep.Buffer.set_num_compute_units(new_num_sms=28)
        assert deep_ep.Buffer.num_sms == 28
        with pytest.raises(TypeError, match="conflicting"):
            deep_ep.Buffer.set_num_sms(new_num_sms=24, new_num_compute_units=26)
    finally:
        deep_ep.Buffer.num_sms = old
    buf = deep_ep.Buffer(None, num_scaleup_bytes=1 << 20, allow_multinode_memory_transport=False,
                         allow_memory_transport_for_low_latency_mode=True)
    assert buf.num_nvl_bytes == 1 << 20
    with pytest.raises(TypeError, match="conflicting"):
        deep_ep.Buffer(None, num_nvl_bytes=128, num_scaleup_bytes=256)
    with pytest.raises(NotImplementedError, match="internode"):
        deep_ep.Buffer(None, num_scaleout_bytes=1 << 20)            # the alias reaches the same rule as num_rdma_bytes
    assert "num_tokens_per_rdma_rank" in inspect.signature(deep_ep.Buffer.dispatch).parameters


def test_elastic_spellings():
    buf = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=8, hidden=64, num_topk=2, num_device_timeout_secs=50,
                                num_host_timeout_secs=40, device="cpu")
    try:
        assert (buf.num_gpu_timeout_secs, buf.num_cpu_timeout_secs) == (50, 40)
        base = buf.get_theoretical_num_sms(256, 8)
        assert buf.get_theoretical_num_compute_units(256, 8) == base
        assert buf.get_theoretical_num_sms(256, 8, scaleup_gbs=900, compute_read_gbs=200, compute_unit_write_gbs=50) == \
            buf.get_theoretical_num_sms(256, 8, nvlink_gbs=900, sm_read_gbs=200, sm_write_gbs=50)
        assert buf.get_theoretical_num_qps(num_compute_units=24) == 0
        with pytest.raises(TypeError, match="conflicting"):
            buf.get_theoretical_num_sms(256, 8, sm_read_gbs=200, compute_read_gbs=100)
    finally:
        buf.destroy()
    with pytest.raises(TypeError, match="conflicting"):
        deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=8, hidden=64, num_topk=2, num_gpu_timeout_secs=100,
                              num_device_timeout_secs=200, device="cpu")
