"""Host-side behaviour: API surface, aliases, layout mirror, store collectives, utils, failure paths without a GPU."""
import inspect
import os
import threading

import pytest
import torch

import deepep_b200 as deep_ep
from deepep_b200 import _compat
from deepep_b200.parallel import layout as L
from deepep_b200.parallel.store import StoreAborted, StoreGroup
from deepep_b200.utils import math as M
from deepep_b200.utils.event import EventHandle, EventOverlap
from deepep_b200.utils.testing import aggregate_rank_max, bandwidth_gbps, nearest_rank


def test_public_exports_and_alias_package():
    assert deep_ep.__all__ == ["Buffer", "ElasticBuffer", "EPHandle", "Config", "EventHandle", "EventOverlap"]
    import deep_ep as alias

    assert alias.ElasticBuffer is deep_ep.ElasticBuffer and alias.Buffer is deep_ep.Buffer
    from deep_ep.utils.math import per_token_cast_to_fp8 as a  # noqa: F401  (submodules resolve through the alias)


def test_signatures_follow_the_upstream_contract():
    init = inspect.signature(deep_ep.ElasticBuffer.__init__).parameters
    for name in ("group", "num_bytes", "num_cpu_bytes", "num_max_tokens_per_rank", "hidden", "num_topk", "use_fp8_dispatch",
                 "deterministic", "allow_hybrid_mode", "allow_multiple_reduction", "prefer_overlap_with_compute", "sl_idx",
                 "num_allocated_qps", "num_cpu_timeout_secs", "num_gpu_timeout_secs", "explicitly_destroy", "rank", "world_size",
                 "bootstrap", "debug_collectives", "machine_type"):
        assert name in init, name
    disp = list(inspect.signature(deep_ep.ElasticBuffer.dispatch).parameters)
    assert disp[:8] == ["self", "x", "topk_idx", "topk_weights", "cumulative_local_expert_recv_stats", "num_experts",
                        "num_max_tokens_per_rank", "expert_alignment"]
    for name in ("previous_event", "async_with_compute_stream", "allocate_on_comm_stream", "handle", "do_handle_copy", "do_cpu_sync",
                 "do_expand", "do_zero_padding", "use_tma_aligned_col_major_sf"):
        assert name in disp
    comb = list(inspect.signature(deep_ep.ElasticBuffer.combine).parameters)
    assert comb[:5] == ["self", "x", "handle", "topk_weights", "bias"]
    handle = list(inspect.signature(deep_ep.EPHandle.__init__).parameters)
    assert handle[1:5] == ["do_expand", "num_experts", "expert_alignment", "num_max_tokens_per_rank"] and handle[-1] == "is_low_latency"
    v1 = list(inspect.signature(deep_ep.Buffer.dispatch).parameters)
    assert v1[:4] == ["self", "x", "handle", "num_tokens_per_rank"] and "num_worst_tokens" in v1


def test_keyword_aliases():
    def f(a, num_sms=0, num_qps=0):
        return a, num_sms, num_qps

    g = _compat.keyword_aliases(f, {"num_compute_units": "num_sms"})
    assert g(1, num_compute_units=4) == (1, 4, 0)
    with pytest.raises(TypeError):
        g(1, num_sms=2, num_compute_units=4)
    h = _compat.public_keywords(f, {"num_units": "num_sms"})
    assert "num_units" in inspect.signature(h).parameters and h(1, num_units=3) == (1, 3, 0)


def test_layout_mirror_and_hints():
    assert L.elastic_size_hint(8, 4096, 7168, 8) % (2 << 20) == 0
    assert L.ll_region_bytes(8, 4096, 7168, 8) == 0 and L.ll_region_bytes(8, 256, 7168, 8) > 0
    with pytest.raises(ValueError):
        L.elastic_size_hint(3, 128, 512, 4)
    with pytest.raises(ValueError):
        L.validate_hidden(100)
    with pytest.raises(ValueError):
        L.validate_hidden(192, fp8=True)
    cfg = deep_ep.Config(24)
    assert cfg.get_nvl_buffer_size_hint(7168 * 2, 8, 4096) > 0 and cfg.get_rdma_buffer_size_hint(1, 1) == 0
    with pytest.raises(ValueError):
        deep_ep.Config(3)


def test_native_layout_matches_python_mirror():
    from deepep_b200.ops import native_available, load_native

    if not native_available():
        pytest.skip("native extension not built")
    C = load_native()
    for a in [(8, 4096, 7168, 8), (2, 128, 512, 4), (1, 100, 256, 2), (4, 16384, 4096, 6)]:
        ll = L.ll_region_bytes(*a)
        assert C.make_layout(*a, ll, 0).total == L.workspace_bytes(*a, ll)
        window = max(1, a[1] // 3)          # a workspace that holds the combine partials of a third of the tokens
        capped = C.make_layout(*a, ll, 0, window)
        assert capped.total == L.workspace_bytes(*a, ll, 0, window) <= C.make_layout(*a, ll, 0).total
        assert capped.partial_tokens == window and C.make_layout(*a, ll, 0).partial_tokens == a[1]
        if ll:
            assert C.ll_region_bytes(a[0], a[1], a[3], a[2]) == ll


def test_fp8_cast_roundtrip_and_helpers():
    x = torch.randn(7, 300).bfloat16()
    q, s = M.per_token_cast_to_fp8(x)
    assert q.shape == x.shape and s.shape == (7, 3)
    back = M.per_token_cast_back(q, s)
    assert (back.float() - x.float()).abs().max() <= x.float().abs().max() * 0.07
    q2, s2 = M.per_token_cast_to_fp8(x, use_ue8m0=True)
    assert torch.equal(torch.exp2(torch.round(torch.log2(s2))), s2)
    t = torch.tensor([[3, 3, -1, 1], [0, 2, 2, 2]])
    M.inplace_unique(t, 4)
    assert t.tolist() == [[3, 1, -1, -1], [2, 0, -1, -1]]
    assert M.calc_diff(x.float(), x.float()) < 1e-12 and M.align(5, 4) == 8 and M.safe_div(0, 0) == 0


def test_events_without_cuda():
    ev = EventOverlap()
    assert ev.event is None
    handle = EventHandle()
    seen = []
    ov = EventOverlap(handle)
    ov.register_hook_after_wait(lambda: seen.append(1) or "done")
    assert ov.wait() == "done" and seen == [1]
    with ov(release_handle=True):
        pass
    assert ov.event is None


def test_bench_statistics():
    stats = aggregate_rank_max([[10, 20, 30, 40], [15, 5, 35, 10]])
    assert stats["mean_rank_max_us"] == (15 + 20 + 35 + 40) / 4 and stats["p50_us"] == 20 and stats["p95_us"] == 40
    assert nearest_rank([1, 2, 3, 4], 0.5) == 2 and bandwidth_gbps(1e9, 1000.0) == 1000.0
    with pytest.raises(ValueError):
        aggregate_rank_max([[1, 2], [1]])


def _store_pair():
    from datetime import timedelta

    from torch.distributed import TCPStore

    server = TCPStore("127.0.0.1", 0, 2, True, timedelta(seconds=20), wait_for_workers=False)
    client = TCPStore("127.0.0.1", server.port, 2, False, timedelta(seconds=20))
    return server, client


def test_store_group_collectives_and_abort():
    server, client = _store_pair()
    groups = [StoreGroup(server, 0, 2, prefix="t", timeout=10), StoreGroup(client, 1, 2, prefix="t", timeout=10)]
    out = [None, None]

    def work(r):
        g = groups[r]
        a = g.all_gather({"rank": r}, "hello")
        g.barrier()
        total = g.reduce_sum([r + 1, 10 * (r + 1)])
        out[r] = (a, total.tolist())

    threads = [threading.Thread(target=work, args=(r,)) for r in range(2)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert out[0] == out[1] == ([{"rank": 0}, {"rank": 1}], [3, 30])
    # a rank that fails tells the others instead of leaving them blocked
    groups[1].abort("boom")
    with pytest.raises(StoreAborted):
        groups[0].all_gather(1, "after")
    with pytest.raises(ValueError):
        StoreGroup(server, 2, 2, prefix="t")


def test_unavailable_features_fail_explicitly():
    with pytest.raises(NotImplementedError):
        deep_ep.Buffer(None, num_rdma_bytes=1)
    with pytest.raises(NotImplementedError):
        deep_ep.Buffer(None, low_latency_mode=True)
    b = deep_ep.Buffer(None)
    with pytest.raises(NotImplementedError):
        b.low_latency_dispatch()
    with pytest.raises(ValueError):
        deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=0, hidden=64, num_topk=2)
    with pytest.raises(ValueError):
        deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=8, hidden=64, num_topk=2, machine_type="global_clos")


def test_native_session_argument_errors_do_not_need_a_gpu():
    from deepep_b200.ops import native_available, load_native

    if not native_available():
        pytest.skip("native extension not built")
    C = load_native()
    before = C.live_instances()
    for bad in [(0, 9, 2 << 20, 10.0), (2, 2, 2 << 20, 10.0), (0, 1, 1000, 10.0), (0, 1, 2 << 20, 0.0)]:
        with pytest.raises(ValueError):
            C.Session(*bad)
    assert C.live_instances() == before            # failed constructors release their instance slot
    with pytest.raises(ValueError):
        C.make_layout(9, 128, 512, 4)
    with pytest.raises(ValueError):
        C.make_layout(2, 128, 511, 4)


def test_failed_workspace_allocation_releases_the_instance_slot():
    """Without a GPU the allocation inside the Session constructor fails: the error surfaces, nothing leaks."""
    from deepep_b200.ops import native_available, load_native

    if not native_available() or torch.cuda.is_available():
        pytest.skip("needs the native extension on a machine without a GPU")
    C = load_native()
    before = C.live_instances()
    with pytest.raises(RuntimeError):
        C.Session(0, 1, 2 << 20, 10.0)
    assert C.live_instances() == before


def test_timeout_environment_override(monkeypatch):
    from deepep_b200.parallel.elastic import _timeout_seconds

    assert _timeout_seconds(100) == 100
    monkeypatch.setenv("DEEPEP_GPU_TIMEOUT_SECONDS", "7")
    assert _timeout_seconds(100) == 7
    monkeypatch.setenv("DEEPEP_GPU_TIMEOUT_SECONDS", "0")
    with pytest.raises(ValueError):
        _timeout_seconds(100)


def test_installation_validator_reports_a_healthy_package():
    """``python -m deepep_b200.validate``: lazy import, binary matches its provenance file, CPU smoke run passes."""
    import json
    import subprocess
    import sys

    from deepep_b200.ops import load_native

    load_native(build_if_missing=True)
    res = subprocess.run([sys.executable, "-m", "deepep_b200.validate"], capture_output=True, text=True, cwd=os.path.dirname(os.path.dirname(__file__)))
    report = json.loads(res.stdout)
    assert res.returncode == 0 and report["ok"] and report["package"]["import_is_lazy"] and report["smoke"]["ok"]


def test_loader_refuses_a_binary_that_is_not_the_recorded_one(tmp_path, monkeypatch):
    import deepep_b200.ops as ops

    monkeypatch.setattr(ops, "_native", None)
    monkeypatch.setattr(ops, "build_info", lambda: {"binary": ops.native_path().name, "binary_sha256": "0" * 64})
    with pytest.raises(ops.NativeUnavailable, match="not the one"):
        ops.load_native()


def test_combine_window_for_a_capped_workspace():
    """Capacity fallback: the largest token window whose combine partials fit the given bytes (bisection), 0 when
    everything fits, an error when not even the fixed regions fit."""
    a = (8, 4096, 7168, 8)
    full = L.elastic_size_hint(*a)
    assert L.combine_window(*a, full) == 0 and L.combine_window(*a, full + 12345) == 0
    ll = L.ll_region_bytes(*a)
    w = L.combine_window(*a, full - (200 << 20))
    assert 0 < w < 4096
    assert L.workspace_bytes(*a, ll, 0, w) <= full - (200 << 20) < L.workspace_bytes(*a, ll, 0, w + 64)
    with pytest.raises(ValueError):
        L.combine_window(*a, 1 << 20)
    buf_args = dict(num_max_tokens_per_rank=64, hidden=256, num_topk=2, explicitly_destroy=True, device="cpu")
    from deepep_b200 import ElasticBuffer
    need = ElasticBuffer.get_buffer_size_hint(None, 64, 256, 2, world_size=1)
    with pytest.raises(ValueError, match="too small"):
        ElasticBuffer(None, num_bytes=4096, **buf_args)
    assert need > 0


def test_numa_binding_reads_sysfs(tmp_path):
    """The NUMA helper parses a node's CPU list from a (fake) sysfs tree, only ever narrows the affinity of this process,
    and answers None where the host gives no information."""
    import os

    from deepep_b200.utils import numa

    assert numa._parse_cpu_list("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert numa.bind_to_numa_node(None) is None
    assert numa.bind_to_numa_node(3, sysfs=str(tmp_path)) is None             # no such node in this tree
    mine = sorted(os.sched_getaffinity(0))
    node = tmp_path / "devices/system/node/node0"
    node.mkdir(parents=True)
    (node / "cpulist").write_text(f"{mine[0]}\n")
    before = os.sched_getaffinity(0)
    try:
        assert numa.bind_to_numa_node(0, sysfs=str(tmp_path)) == {mine[0]}
        assert os.sched_getaffinity(0) == {mine[0]}
        (node / "cpulist").write_text("100000\n")                              # a CPU this process may not use: unchanged
        assert numa.bind_to_numa_node(0, sysfs=str(tmp_path)) is None and os.sched_getaffinity(0) == {mine[0]}
    finally:
        os.sched_setaffinity(0, before)
