"""High-throughput notify/dispatch/combine kernels, N virtual ranks on one GPU, against the CPU oracle."""
import pytest
import torch

from deepep_b200.oracle import reference as R
from helpers import bits_equal, make_routes, make_weights

pytestmark = pytest.mark.gpu


def run_case(world, tokens, hidden, experts, topk, mode, *, expand=True, alignment=1, dmode=0, seed=0, max_tokens=None,
             with_bias=False, repeats=1, local_direct=True):
    from deepep_b200.parallel.virtual import VirtualWorld

    dev = torch.device("cuda")
    max_tokens = max_tokens or max(tokens)
    xs = [torch.randn((t, hidden), generator=torch.Generator().manual_seed(seed + r)).bfloat16() for r, t in enumerate(tokens)]
    idx = [make_routes(mode, t, experts, topk, world, seed + 10 * r) for r, t in enumerate(tokens)]
    wts = [make_weights(t, topk, seed + r) for r, t in enumerate(tokens)]
    with VirtualWorld(world, max_tokens, hidden, topk, timeout=10.0) as vw:
        eng = vw.engine
        eng.local_direct = local_direct   # False: rows that stay on their rank also go through staging / partial areas
        for rep in range(repeats):
            plans = eng.notify([i.to(dev) for i in idx], [w.to(dev) for w in wts], experts, expand=expand, alignment=alignment)
            if dmode == 1:
                from deepep_b200.utils.math import per_token_cast_to_fp8
                q = [per_token_cast_to_fp8(x) for x in xs]
                dev_x = [(a.to(dev), b.to(dev)) for a, b in q]
                ref_x = q
            else:
                dev_x = [x.to(dev) for x in xs]
                ref_x = xs
            outs = eng.dispatch(dev_x, plans, dmode)
            ref, lays = R.dispatch(ref_x, idx, wts, experts, do_expand=expand, expert_alignment=alignment,
                                   quantize_fp8=(dmode == 2))
            torch.cuda.synchronize()
            eng.check_status()
            for r in range(world):
                (rx, rsf), plan, lay = outs[r], plans[r], lays[r]
                assert plan.num_rows == lay.num_rows, (r, plan.num_rows, lay.num_rows)
                assert plan.expert_counts_list == lay.expert_counts.tolist()
                exp_x = ref[r][0]
                if dmode == 0:
                    assert bits_equal(rx, exp_x), f"rank {r} payload differs"
                else:
                    valid = lay.row_index
                    assert bits_equal(rx.cpu()[valid], exp_x[0][valid]), f"rank {r} fp8 payload differs"
                    assert bits_equal(rsf.cpu()[valid], exp_x[1][valid]), f"rank {r} scales differ"
                if expand:
                    assert torch.equal(plan.recv_w[:plan.num_rows].cpu(), ref[r][2])
                else:
                    assert torch.equal(plan.recv_idx[:plan.num_rows].cpu(), ref[r][1])
                    assert torch.equal(plan.recv_w[:plan.num_rows].cpu(), ref[r][2])
            # combine: expert output = received row scaled by a per-row factor (bf16), value channel = 0.5 - w
            eouts, evals = [], []
            for r in range(world):
                rx = outs[r][0] if dmode == 0 else None
                base = ref[r][0] if dmode == 0 else None
                if dmode != 0:
                    base = torch.randn((lays[r].num_rows, hidden), generator=torch.Generator().manual_seed(99 + r)).bfloat16()
                eo = (base.float() * 0.5).bfloat16()
                eouts.append(eo)
                evals.append(0.5 - ref[r][2])
            bias = None
            if with_bias:
                bias = [(torch.randn((t, hidden), generator=torch.Generator().manual_seed(5 + r)).bfloat16(),
                         torch.randn((t, hidden), generator=torch.Generator().manual_seed(6 + r)).bfloat16()) for r, t in enumerate(tokens)]
            couts = eng.combine([e.to(dev) for e in eouts], plans, [v.to(dev) for v in evals],
                                bias=None if bias is None else [(a.to(dev), b.to(dev)) for a, b in bias])
            cref = R.combine(eouts, lays, tokens, topk, topk_weights=evals, bias=bias)
            torch.cuda.synchronize()
            eng.check_status()
            for r in range(world):
                assert bits_equal(couts[r][0], cref[r][0]), f"rank {r} combined payload differs"
                assert torch.equal(couts[r][1].cpu(), cref[r][1]), f"rank {r} returned weights differ"


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("mode", ["random", "invalid"])
def test_expand_bf16(world, mode):
    run_case(world, [100] * world, 512, 16 * world if world < 8 else 64, 4, mode)


def test_uneven_tokens_and_empty_rank():
    run_case(4, [130, 0, 64, 7], 256, 32, 6, "empty", repeats=2)


def test_alignment_padding():
    run_case(2, [96, 80], 512, 16, 4, "random", alignment=8)


def test_rank_layout():
    run_case(4, [70, 90, 64, 65], 512, 32, 4, "invalid", expand=False)


def test_fp8_given_and_fused():
    run_case(2, [128, 100], 1024, 16, 4, "random", dmode=1)
    run_case(2, [128, 100], 1024, 16, 4, "random", dmode=2)
    run_case(2, [50, 60], 384, 16, 4, "random", dmode=1)   # scale rows not 16-byte aligned


@pytest.mark.parametrize("world", [1, 2, 4])
def test_local_rows_through_staging(world):
    """The same results when a rank's own rows take the staging area and the partial area like remote rows."""
    run_case(world, [100, 77, 64, 130][:world], 512, 16 * world, 4, "invalid", local_direct=False, repeats=2)
    run_case(world, [100, 77, 64, 130][:world], 512, 16 * world, 4, "random", expand=False, local_direct=False)


def test_rank_layout_fp8_and_bias():
    run_case(2, [90, 120], 1024, 16, 4, "random", expand=False, dmode=1, with_bias=True)
    run_case(1, [200], 1024, 8, 4, "invalid", expand=False, dmode=2)


def test_bias_and_hotspot():
    run_case(4, [128] * 4, 1024, 32, 8, "hotspot", with_bias=True)


def test_large_hidden_repeat():
    run_case(2, [300, 280], 7168, 64, 8, "random", repeats=3)


def test_wait_timeout_reports_status():
    """A wait on a flag nobody writes runs out, the kernel returns, the host sees TIMEOUT."""
    from deepep_b200.parallel.virtual import VirtualWorld
    from deepep_b200.parallel.engine_cuda import CommunicationError

    with VirtualWorld(1, 64, 256, 2, timeout=0.005) as vw:
        s = vw.sessions[0]
        s.wait_probe(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        st = s.status()
        assert st["code"] == 1 and st["where"] == 99
        with pytest.raises(CommunicationError):
            vw.engine.check_status()
        s.clear_status()
        torch.cuda.synchronize()
        assert s.status()["code"] == 0


def test_workspace_canary_detects_overrun():
    """The allocation ends in a canary zone: intact after real work, reported once something writes behind the workspace."""
    from deepep_b200.models.mega_moe import _view
    from deepep_b200.ops import load_native

    C = load_native()
    layout = C.make_layout(1, 64, 256, 2, 0, 0)
    s = C.Session(0, 1, layout.total, 5.0)
    try:
        assert s.guard_intact()
        _view(s.workspace + s.bytes - 16, 16, torch.device("cuda")).fill_(7)        # last bytes of the workspace proper
        torch.cuda.synchronize()
        assert s.guard_intact()
        _view(s.workspace + s.bytes, 8, torch.device("cuda")).zero_()               # first bytes of the canary zone
        torch.cuda.synchronize()
        assert not s.guard_intact()
    finally:
        s.close()


def test_index_checks_report_instead_of_reading_out_of_range():
    """Only in a build with DEEPEP_DEBUG_BOUNDS=1: a combine whose input has fewer rows than the routing plan names is
    reported through the status block and the rows are not read.  (The short input is a view of a full-size
    allocation, so nothing is out of range of the allocation either way.)"""
    from deepep_b200.ops import load_native
    from deepep_b200.parallel.engine_cuda import CommunicationError
    from deepep_b200.parallel.virtual import VirtualWorld

    if not load_native().debug_bounds:
        pytest.skip("needs a build with DEEPEP_DEBUG_BOUNDS=1")
    dev = torch.device("cuda")
    T, H, E, K = 64, 256, 4, 2
    x = torch.randn((T, H)).bfloat16().to(dev)
    idx = make_routes("random", T, E, K, 1, 0).to(dev)
    vw = VirtualWorld(1, T, H, K, timeout=5.0)
    try:
        plans = vw.engine.notify([idx], [None], E)
        rows = vw.engine.dispatch([x], plans, 0)[0][0]
        short = rows[: rows.shape[0] // 2]
        vw.engine.combine([short], plans, [None])
        torch.cuda.synchronize()
        with pytest.raises(CommunicationError):
            vw.engine.check_status()
        status = vw.sessions[0].status()
        assert status["code"] == 2 and status["where"] == 100 and status["expected"] == short.shape[0]
    finally:
        torch.cuda.synchronize()
        for s in vw.sessions:
            s.close()


def test_combine_in_token_windows():
    """Capacity fallback: the workspace holds the combine partials of 48 tokens at a time, so the combine of up to 200
    tokens per rank runs as five passes (one launch per window) and must still match the oracle bit for bit."""
    from deepep_b200.parallel.virtual import VirtualWorld

    dev = torch.device("cuda")
    world, tokens, hidden, experts, topk = 4, [130, 64, 1, 200], 512, 16, 4
    xs = [torch.randn((t, hidden), generator=torch.Generator().manual_seed(r)).bfloat16() for r, t in enumerate(tokens)]
    idx = [make_routes("invalid", t, experts, topk, world, 10 * r) for r, t in enumerate(tokens)]
    wts = [make_weights(t, topk, r) for r, t in enumerate(tokens)]
    ref, lays = R.dispatch(xs, idx, wts, experts, do_expand=True)
    eouts = [(ref[r][0].float() * 0.5).bfloat16() for r in range(world)]
    evals = [0.5 - ref[r][2] for r in range(world)]
    cref = R.combine(eouts, lays, tokens, topk, topk_weights=evals)
    for local_direct in (True, False):
        with VirtualWorld(world, max(tokens), hidden, topk, timeout=10.0, partial_tokens=48) as vw:
            eng = vw.engine
            eng.local_direct = local_direct
            assert vw.layout.partial_tokens == 48
            plans = eng.notify([i.to(dev) for i in idx], [w.to(dev) for w in wts], experts, expand=True, alignment=1)
            outs = eng.dispatch([x.to(dev) for x in xs], plans, 0)
            for rep in range(2):
                couts = eng.combine([e.to(dev) for e in eouts], plans, [v.to(dev) for v in evals])
                torch.cuda.synchronize()
                eng.check_status()
                for r in range(world):
                    assert bits_equal(outs[r][0], ref[r][0])
                    assert bits_equal(couts[r][0], cref[r][0]), f"rank {r} combined payload differs"
                    assert torch.equal(couts[r][1].cpu(), cref[r][1]), f"rank {r} returned weights differ"


def test_public_api_with_a_capped_workspace():
    """``num_bytes`` below the size hint: the buffer picks the largest token window that fits and combine still matches."""
    from deepep_b200 import ElasticBuffer
    from deepep_b200.parallel import layout as L

    dev = torch.device("cuda")
    T, H, E, K = 1024, 2048, 32, 6
    need = ElasticBuffer.get_buffer_size_hint(None, T, H, K, world_size=1)
    cap = need - (2 << 20)                  # 2 MiB short of the 4 MiB of partials: about half of the tokens fit at a time
    buf = ElasticBuffer(None, num_bytes=cap, num_max_tokens_per_rank=T, hidden=H, num_topk=K, explicitly_destroy=True)
    assert 0 < buf.combine_window < T and buf.num_bytes <= cap
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(1)).bfloat16()
    idx = make_routes("random", T, E, K, 1, 3)
    w = make_weights(T, K, 2)
    rx, _, rw, handle, _ = buf.dispatch(x.to(dev), topk_idx=idx.to(dev), topk_weights=w.to(dev), num_experts=E, do_expand=True)
    ref, lays = R.dispatch([x], [idx], [w], E, do_expand=True)
    assert bits_equal(rx, ref[0][0])
    out, _, _ = buf.combine(rx, handle)
    assert bits_equal(out, R.combine([ref[0][0]], lays, [T], K)[0][0])
    buf.destroy()


def test_phase_stamps_of_the_profile_instantiations():
    """`enable_device_profile` launches the profile instantiations; the routing pass stamps its phases (monotonic,
    microseconds) and the high-throughput kernels fill one record per block.  Production launches leave no stamps."""
    from deepep_b200.parallel.virtual import VirtualWorld

    dev = torch.device("cuda")
    world, T, H, E, K = 2, 96, 256, 8, 2
    xs = [torch.randn((T, H), generator=torch.Generator().manual_seed(r)).bfloat16().to(dev) for r in range(world)]
    idx = [make_routes("random", T, E, K, world, r).to(dev) for r in range(world)]
    wts = [make_weights(T, K, r).to(dev) for r in range(world)]
    with VirtualWorld(world, T, H, K, timeout=10.0) as vw:
        eng = vw.engine
        eng.enable_device_profile(True)
        plans = eng.notify(idx, wts, E, expand=True, alignment=1)
        outs = eng.dispatch(xs, plans, 0)
        eng.combine([o[0] for o in outs], plans, [None] * world)
        stamps = eng.phase_stamps("notify")
        order = [stamps[k] for k in ("table_sent", "tables_in", "histograms", "scans", "records", "done")]
        assert all(b >= a for a, b in zip(order, order[1:])) and 0 < order[-1] < 1e5, stamps
        prof = eng.pop_device_profile()
        assert {op for op, _ in prof} == {"dispatch", "combine"}
        for blocks in prof.values():
            assert blocks and all(b["end_us"] >= b["start_us"] >= 0 for b in blocks) and sum(b["rows"] for b in blocks) > 0
        eng.enable_device_profile(False)
        eng.check_status()
