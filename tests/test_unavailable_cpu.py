"""Operations this library declares but does not provide fail with an explicit ``NotImplementedError`` before they touch
their inputs (the reference tests the same property of its own unavailable operations, ``tests/api/test_unavailable.py``)."""
import pytest


class Untouchable:
    """Any attribute access, call or conversion of an argument is a test failure."""

    def __getattr__(self, name):
        raise AssertionError(f"the unavailable operation inspected its argument ({name})")

    def __bool__(self):
        raise AssertionError("the unavailable operation inspected its argument")


ELASTIC = ["engram_write", "engram_fetch", "pp_set_config", "pp_send", "pp_recv"]
V1 = ["internode_dispatch", "internode_combine", "clean_low_latency_buffer", "low_latency_dispatch", "low_latency_combine",
      "get_next_low_latency_combine_buffer"]


@pytest.mark.parametrize("method", ELASTIC)
def test_elastic_buffer_out_of_scope_operations(method):
    from deepep_b200 import ElasticBuffer

    buf = ElasticBuffer(None, num_max_tokens_per_rank=16, hidden=128, num_topk=2, explicitly_destroy=True, device="cpu")
    try:
        with pytest.raises(NotImplementedError, match="outside the scope"):
            getattr(buf, method)(Untouchable(), Untouchable(), key=Untouchable())
    finally:
        buf.destroy()


@pytest.mark.parametrize("method", V1)
def test_v1_buffer_unavailable_operations(method):
    from deepep_b200 import Buffer

    with pytest.raises(NotImplementedError):
        getattr(Buffer, method)(Untouchable(), Untouchable(), Untouchable())


@pytest.mark.parametrize("kwargs, message", [
    (dict(num_rdma_bytes=1 << 20), "internode"),
    (dict(low_latency_mode=True), "low-latency"),
    (dict(enable_shrink=True), "shrinking"),
])
def test_v1_constructor_rejects_modes_without_a_counterpart(kwargs, message):
    from deepep_b200 import Buffer

    with pytest.raises(NotImplementedError, match=message):
        Buffer(None, **kwargs)
