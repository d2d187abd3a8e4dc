"""The upstream-compatible helpers (``deep_ep.utils``) and the small static parts of the V1 ``Buffer`` on the CPU.

Parity: ``deep_ep/utils/math.py`` and ``deep_ep/utils/testing.py`` of the reference; expectations below are calculated
by hand or by an independent formulation.
"""
import pytest
import torch

import deepep_b200 as deep_ep
from deepep_b200.utils import math as M
from deepep_b200.utils import testing as TU


def test_fp8_casts_round_trip():
    g = torch.Generator().manual_seed(1)
    x = (torch.randn((5, 300), generator=g) * 3).bfloat16()            # 300 is not a multiple of 128: the tail block is padded
    q, scale = M.per_token_cast_to_fp8(x)
    assert q.dtype == torch.float8_e4m3fn and q.shape == x.shape and scale.shape == (5, 3) and scale.dtype == torch.float32
    amax = torch.stack([x[:, i * 128:(i + 1) * 128].abs().float().amax(1) for i in range(3)], 1).clamp(1e-4)
    assert torch.equal(scale, amax / 448.0)
    back = M.per_token_cast_back(q, scale)
    assert back.dtype == torch.bfloat16 and M.calc_diff(back.float(), x.float()) < 1e-3
    # power-of-two scales: never smaller than the exact ones, exact in ue8m0, and the packed-exponent form reads back alike
    q2, scale2 = M.per_token_cast_to_fp8(x, use_ue8m0=True)
    mantissa, exponent = torch.frexp(scale2)
    assert bool((mantissa == 0.5).all()) and bool((scale2 >= scale).all()) and bool((scale2 < 2 * scale + 1e-30).all())
    packed = torch.zeros((5, 4), dtype=torch.uint8)
    packed[:, :3] = (exponent - 1 + 127).to(torch.uint8)
    as_int = (packed.view(torch.int32))                                                 # four codes per int32, as upstream packs them
    full = torch.zeros((5, 512), dtype=torch.float8_e4m3fn)
    full.view(torch.uint8)[:, :300] = q2.view(torch.uint8)
    via_int = M.per_token_cast_back(full, as_int)
    direct = M.per_token_cast_back(q2, scale2)
    assert torch.equal(via_int[:, :300], direct)
    empty = M.per_token_cast_to_fp8(x[:0])
    assert empty[0].shape == (0, 300) and empty[1].shape == (0, 3) and M.per_token_cast_back(*empty).shape == (0, 300)


def test_small_math_helpers():
    assert M.ceil_div(7, 3) == 3 and M.align(7, 4) == 8 and M.align(8, 4) == 8
    assert M.safe_div(0, 0) == 0 and M.safe_div(3, 2) == 1.5
    with pytest.raises(ZeroDivisionError):
        M.safe_div(1, 0)
    assert M.calc_diff(torch.ones(4), torch.ones(4)) == pytest.approx(0.0, abs=1e-12)
    assert M.calc_diff(torch.zeros(4), torch.ones(4)) == pytest.approx(1 - 2 * 8 / (4 + 16))
    ids = torch.tensor([[3, 3, -1, 0], [-1, -1, -1, -1], [5, 1, 5, 2]])
    M.inplace_unique(ids, 6)
    assert ids.tolist() == [[3, 0, -1, -1], [-1, -1, -1, -1], [5, 2, 1, -1]]
    scores = torch.arange(1, 13, dtype=torch.float32).view(2, 6)         # 3 groups of 2 experts
    kept = M.create_grouped_scores(scores, torch.tensor([[0, 2], [1, 1]]), 3)
    assert kept.tolist() == [[1, 2, 0, 0, 5, 6], [0, 0, 9, 10, 0, 0]]
    a, b = torch.tensor([1, 2, 3], dtype=torch.int32), torch.tensor([[4.0]], dtype=torch.float32)
    assert M.hash_tensor(a) == 6 and M.hash_tensors(a, (a, None), b) == M.hash_tensor(b)      # equal hashes cancel under xor
    assert M.count_bytes(a, None, (b, [a])) == 12 + 4 + 12


def test_timing_aggregation():
    assert TU.nearest_rank([1.0, 2.0, 3.0, 4.0], 0.5) == 2.0 and TU.nearest_rank([1.0, 2.0, 3.0, 4.0], 0.95) == 4.0
    assert TU.nearest_rank([7.0], 0.0) == 7.0
    with pytest.raises(ValueError, match="no samples"):
        TU.nearest_rank([], 0.5)
    agg = TU.aggregate_rank_max([[10.0, 30.0, 20.0], [12.0, 25.0, 50.0]])         # per-iteration maximum: 12, 30, 50
    assert agg == {"mean_rank_max_us": pytest.approx(92 / 3), "min_us": 12.0, "max_us": 50.0, "p50_us": 30.0, "p95_us": 50.0,
                   "iterations": 3}
    with pytest.raises(ValueError, match="same number"):
        TU.aggregate_rank_max([[1.0], [1.0, 2.0]])
    assert TU.bandwidth_gbps(2e9, 1000.0) == pytest.approx(2000.0) and TU.bandwidth_gbps(1.0, 0.0) == 0.0
    TU.flush_l2_cache()                                                          # nothing to flush without a GPU
    with pytest.raises(ValueError, match="at least two"):
        TU.bench(lambda: None, num_tests=1)
    with pytest.raises(ValueError, match="greater than or equal"):
        TU.bench(lambda: None, num_warmups=-1)


def test_v1_buffer_static_parts():
    Buffer, Config = deep_ep.Buffer, deep_ep.Config
    old = Buffer.num_sms
    try:
        Buffer.set_num_sms(24)
        assert Buffer.num_sms == 24 and Buffer.get_dispatch_config(8).num_sms == 24 and Buffer.get_combine_config(8).num_sms == 24
        for bad in (0, 7, -2):
            with pytest.raises(ValueError, match="even"):
                Buffer.set_num_sms(bad)
    finally:
        Buffer.num_sms = old
    assert isinstance(Buffer.capture(), deep_ep.EventOverlap) and Buffer.capture().event is not None
    hint = Buffer.get_low_latency_rdma_size_hint(128, 7168, 8, 256)
    assert hint == deep_ep.ElasticBuffer.get_buffer_size_hint(None, 128, 7168, 8, world_size=8) and hint % (2 << 20) == 0
    cfg = Config(20)
    assert cfg.get_rdma_buffer_size_hint(14336, 8) == 0 and cfg.get_nvl_buffer_size_hint(14336, 8, 4096) % (2 << 20) == 0
    for args, message in (((21,), "even"), ((20, 0, 256), "positive"), ((20, 256, 256), "smaller")):
        with pytest.raises(ValueError, match=message):
            Config(*args)


def test_v1_buffer_argument_errors():
    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    buf = deep_ep.Buffer(None, num_max_tokens_per_rank=32, hidden=64, num_topk=2)
    assert buf.get_comm_stream() is None
    x, idx = torch.zeros((4, 64), dtype=torch.bfloat16), torch.tensor([[0, 1], [2, 3], [1, -1], [-1, -1]])
    per_expert = buf.get_dispatch_layout(idx, 4)[2]
    with pytest.raises(ValueError, match="contiguous int64"):
        buf.get_dispatch_layout(idx.to(torch.int32), 4)
    with pytest.raises(ValueError, match="multiple of the world size"):
        buf.get_dispatch_layout(idx, 0)
    with pytest.raises(ValueError, match="positive"):
        buf.dispatch(x, topk_idx=idx, num_tokens_per_expert=per_expert, expert_alignment=0)
    with pytest.raises(ValueError, match="get_dispatch_layout"):
        buf.dispatch(x, topk_idx=idx)
    with pytest.raises(TypeError, match="Buffer.dispatch"):
        buf.dispatch(x, handle=("not", "a", "handle"))
    with pytest.raises(TypeError, match="Buffer.dispatch"):
        buf.combine(x, ("not", "a", "handle"))
    with pytest.raises(ValueError, match="another"):
        buf.dispatch(torch.zeros((4, 128), dtype=torch.bfloat16), topk_idx=idx, num_tokens_per_expert=per_expert)
    rx, _, _, _, handle, _ = buf.dispatch(x, topk_idx=idx, num_tokens_per_expert=per_expert)
    with pytest.raises(ValueError):                                       # wrong row count: the slot returns to DISPATCH_READY
        buf.combine(torch.zeros((rx.shape[0] + 1, 64), dtype=torch.bfloat16), handle)
    assert handle.slot.state is deep_ep.SlotState.DISPATCH_READY
    out, _, _ = buf.combine(rx, handle)
    assert out.shape == x.shape
    buf.destroy()
    fresh = deep_ep.Buffer(None)
    with pytest.raises(RuntimeError, match="produced the handle"):
        fresh.combine(x, handle)


def test_bench_kineto_argument_rules():
    """The profiler-based timer checks its arguments before it touches a device."""
    for names, kind in ((5, TypeError), ((), TypeError), (("a", 3), TypeError), (("a", ""), ValueError)):
        with pytest.raises(kind):
            TU.bench_kineto(lambda: None, names)
    with pytest.raises(ValueError, match="num_tests"):
        TU.bench_kineto(lambda: None, "kernel", num_tests=0)
    with pytest.raises(ValueError, match="num_kernels_per_period"):
        TU.bench_kineto(lambda: None, "kernel", num_kernels_per_period=0)


def test_event_overlap_accepts_a_duck_typed_event():
    """Any object with ``current_stream_wait`` serves as the event; the hook's result comes back from the wait."""
    from deepep_b200.utils.event import EventHandle, EventOverlap

    class Mine:
        waits = 0

        def current_stream_wait(self):
            self.waits += 1

    mine = Mine()
    overlap = EventOverlap(mine, extra_tensors=(torch.zeros(2),))
    overlap.register_hook_after_wait(lambda: "epilogue")
    assert overlap.wait() == "epilogue" and mine.waits == 1 and overlap.wait() is None and mine.waits == 2
    with overlap(release_handle=True):
        pass
    assert overlap.event is None and mine.waits == 3 and overlap.extra_tensors is not None
    handle = EventHandle()
    assert handle.query() and handle.device is None and handle.stream is None
    handle.synchronize()


def test_event_overlap_failure_paths_keep_state():
    """A hook that raises stays registered and nothing is released, so the wait can be retried; the wait at the end of
    a ``with`` block also runs when the body raised.  Parity: ``tests/runtime/test_runtime.py:85-92,154-170`` there."""
    from deepep_b200.utils.event import EventOverlap

    class Mine:
        waits = 0

        def current_stream_wait(self):
            self.waits += 1

    attempts = []

    def hook():
        attempts.append(1)
        if len(attempts) == 1:
            raise ValueError("epilogue failed")
        return 7

    overlap = EventOverlap(Mine())
    overlap.register_hook_after_wait(hook)
    with pytest.raises(ValueError, match="epilogue"):
        overlap.current_stream_wait(True)
    assert overlap.event is not None and overlap.hook_after_wait is hook
    assert overlap.current_stream_wait(True) == 7 and overlap.event is None and overlap.hook_after_wait is None
    mine = Mine()
    other = EventOverlap(mine)
    with pytest.raises(KeyError):
        with other(True):
            raise KeyError("body")
    assert mine.waits == 1 and other.event is None
