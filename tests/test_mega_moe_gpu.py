"""Fused MoE forward (route -> GEMM1 + SwiGLU/requant -> GEMM2 + combine -> weighted reduce) against the CPU oracle."""
import pytest
import torch

from deepep_b200.oracle import megamoe as O
from helpers import make_routes, make_weights

pytestmark = pytest.mark.gpu


def _mixed_error_ok(actual, expected, diff_thd=0.01, pct_thd=0.05, max_diff=0.1):
    """The reference's mixed-error gate: few elements beyond diff_thd (abs or rel), none beyond max_diff."""
    a, e = actual.float(), expected.float()
    diff = (a - e).abs()
    rel = diff / e.abs().clamp(min=1.0)
    bad = (rel > diff_thd).float().mean().item()
    return bad <= pct_thd and rel.max().item() <= max_diff, bad, rel.max().item()


def _case(world, tokens, H, I, E, K, seed=0, interleave=None, pairs=None):
    from deepep_b200.models.mega_moe import MegaEngine, transform_weights_for_mega_moe
    from deepep_b200.ops import load_native
    from deepep_b200.parallel.virtual import VirtualWorld

    C = load_native()
    dev = torch.device("cuda")
    M = max(tokens)
    L = E // world
    l1, l2 = O.make_weights(E, H, I, seed)
    xs, idx, ws = [], [], []
    for r, t in enumerate(tokens):
        x = torch.randn((t, H), generator=torch.Generator().manual_seed(seed + r))
        xs.append(O.quantize_mxfp8(x))
        idx.append(make_routes("invalid" if r % 2 else "random", t, E, K, world, seed + 10 * r))
        ws.append(make_weights(t, K, seed + r))
    ref = O.mega_moe_reference(xs, idx, ws, l1, l2, E)
    mega = MegaEngine.mega_bytes(C, M, H, K)
    layout = C.make_mega_layout(world, M, H, K, mega)
    sessions = [C.Session(r, world, layout.total, 20.0) for r in range(world)]
    for s in sessions:
        s.attach_peers([q.workspace for q in sessions])
    try:
        eng = MegaEngine(sessions, layout, dev, E, I)
        if interleave is not None:
            eng.interleave = interleave
        if pairs is not None:
            eng.pairs = pairs
        w = [transform_weights_for_mega_moe((l1[0][r * L:(r + 1) * L], l1[1][r * L:(r + 1) * L]),
                                            (l2[0][r * L:(r + 1) * L], l2[1][r * L:(r + 1) * L]), device=dev) for r in range(world)]
        ys = [torch.zeros((t, H), dtype=torch.bfloat16, device=dev) for t in tokens]
        for rep, fused in enumerate((True, False, True)):
            for r, t in enumerate(tokens):
                x, sf, ti, tw = eng.input_views(r)
                x[:t].copy_(xs[r][0]); sf[:t].copy_(xs[r][1]); ti[:t].copy_(idx[r].to(torch.int32)); tw[:t].copy_(ws[r])
            for y in ys:
                y.zero_()
            eng.forward(ys, tokens, [a for a, _ in w], [b for _, b in w], fused=fused)
            torch.cuda.synchronize()
            eng.check()
            for s in sessions:
                assert s.status()["code"] == 0, s.status()
            for r in range(world):
                ok, bad, worst = _mixed_error_ok(ys[r].cpu(), ref[r])
                assert ok, f"rank {r} (fused={fused}): {bad:.4f} of elements off, worst relative error {worst:.4f}"
    finally:
        torch.cuda.synchronize()
        for s in sessions:
            s.close()


def test_single_rank_small():
    _case(1, [64], 256, 128, 4, 2)


def test_two_virtual_ranks():
    _case(2, [100, 77], 512, 256, 8, 4)


def test_four_virtual_ranks_topk8():
    _case(4, [128, 64, 1, 130], 1024, 256, 32, 8, seed=5)


def test_interleaved_schedule_on_many_row_blocks():
    """Enough row blocks (48+) for the wave schedule to really interleave GEMM1 and GEMM2 tiles (waves of 19 blocks)."""
    _case(1, [768], 512, 2048, 8, 8, seed=9, interleave=1)


def test_cta_pairs_in_the_fused_kernel():
    """The fused kernel as clusters of two CTAs that share every weights tile (tcgen05.mma.cta_group::2): experts are
    padded to whole pairs of row blocks, odd tile counts and empty experts included."""
    _case(1, [300], 256, 128, 4, 2, seed=2, pairs="1")
    _case(1, [768], 512, 2048, 8, 8, seed=9, pairs="1")


def test_shared_experts_stats_bf16_input_and_timer():
    """Public API on one rank: two shared experts, cumulative receive statistics, bf16 activations quantised inside the
    kernel, the reference's call signature (returns None, batch = y.shape[0]) and the phase timer."""
    from deepep_b200.models import mega_tools as MT
    from deepep_b200.models.mega_moe import SymmBuffer, fp8_fp4_mega_moe, mega_moe, transform_weights_for_mega_moe

    dev = torch.device("cuda")
    T, H, I, E, K, S = 200, 512, 256, 8, 4, 2
    l1, l2 = O.make_weights(E, H, I, 3)
    sl1, sl2 = O.make_weights(S, H, I, 100003)
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(1)).bfloat16()
    idx, w = make_routes("invalid", T, E, K, 1, 7), make_weights(T, K, 2)
    ref = O.mega_moe_reference([O.quantize_mxfp8(x)], [idx], [w], l1, l2, E, sl1, sl2)[0]
    buf = SymmBuffer(None, E, 256, K, H, I, num_shared_experts=S)
    try:
        w1, w2 = transform_weights_for_mega_moe(l1, l2, device=dev)
        sw1, sw2 = transform_weights_for_mega_moe(sl1, sl2, device=dev)
        buf.topk_idx[:T].copy_(idx.to(torch.int32)); buf.topk_weights[:T].copy_(w)
        stats = torch.zeros(E, dtype=torch.int32, device=dev)
        timer = buf.allocate_timer()
        y = torch.zeros((T, H), dtype=torch.bfloat16, device=dev)
        for rep in range(2):
            assert fp8_fp4_mega_moe(y, w1, w2, buf, sw1, sw2, stats, x=x.to(dev), timer=timer, check=True) is None
        ok, bad, worst = _mixed_error_ok(y.cpu(), ref)
        assert ok, f"{bad:.4f} of elements off, worst relative error {worst:.4f}"
        # the in-kernel quantiser wrote exactly the oracle's codes and scales into the symmetric inputs
        codes, sf = O.quantize_mxfp8(x)
        assert torch.equal(buf.x[:T].view(torch.uint8).cpu(), codes.view(torch.uint8)) and torch.equal(buf.x_sf[:T].cpu(), sf)
        counts = torch.bincount(idx[idx >= 0].flatten(), minlength=E).int()
        assert torch.equal(stats.cpu(), 2 * counts)                         # two calls accumulated
        phases = MT.parse_timer(timer)
        assert phases["ctas"] > 0 and phases["total_us"] > 0
        assert all(phases[k] >= 0 for k in ("handshake_us", "layout_us", "gemm_us", "finish_sync_us", "reduce_us"))
        # pre-quantised inputs through the convenience wrapper give the same rows
        y2, per_call = mega_moe((codes.to(dev), sf.to(dev)), idx.to(dev), w.to(dev), w1, w2, buf, shared_l1_weights=sw1,
                                shared_l2_weights=sw2)
        torch.cuda.synchronize()
        assert torch.equal(y2, y) and torch.equal(per_call.cpu(), counts)       # the rows of this call alone
        with pytest.raises(ValueError, match="shared"):
            fp8_fp4_mega_moe(y, w1, w2, buf)                                # the buffer was built for two shared experts
    finally:
        buf.destroy()


def test_shared_experts_on_two_virtual_ranks():
    """Shared experts next to routed ones on two ranks (engine level): rows of the shared experts never leave their rank."""
    from deepep_b200.models.mega_moe import MegaEngine, MegaWeights, transform_weights_for_mega_moe
    from deepep_b200.ops import load_native

    C = load_native()
    dev = torch.device("cuda")
    world, tokens, H, I, E, K, S = 2, [90, 130], 512, 256, 8, 4, 1
    L = E // world
    l1, l2 = O.make_weights(E, H, I, 11)
    sl1, sl2 = O.make_weights(S, H, I, 100011)
    xs = [O.quantize_mxfp8(torch.randn((t, H), generator=torch.Generator().manual_seed(20 + r))) for r, t in enumerate(tokens)]
    idx = [make_routes("random", t, E, K, world, 30 + r) for r, t in enumerate(tokens)]
    ws = [make_weights(t, K, 40 + r) for r, t in enumerate(tokens)]
    ref = O.mega_moe_reference(xs, idx, ws, l1, l2, E, sl1, sl2)
    M = max(tokens)
    layout = C.make_mega_layout(world, M, H, K, MegaEngine.mega_bytes(C, M, H, K, S))
    sessions = [C.Session(r, world, layout.total, 20.0) for r in range(world)]
    for s in sessions:
        s.attach_peers([q.workspace for q in sessions])
    try:
        eng = MegaEngine(sessions, layout, dev, E, I, num_shared_experts=S)
        sw = transform_weights_for_mega_moe(sl1, sl2, device=dev)
        w1s, w2s = [], []
        for r in range(world):
            a, b = transform_weights_for_mega_moe((l1[0][r * L:(r + 1) * L], l1[1][r * L:(r + 1) * L]),
                                                  (l2[0][r * L:(r + 1) * L], l2[1][r * L:(r + 1) * L]), device=dev)
            w1s.append(MegaWeights(torch.cat([a.packed, sw[0].packed]), torch.cat([a.sf_chunks, sw[0].sf_chunks]), L + S, a.n, a.k))
            w2s.append(MegaWeights(torch.cat([b.packed, sw[1].packed]), torch.cat([b.sf_chunks, sw[1].sf_chunks]), L + S, b.n, b.k))
        ys = [torch.zeros((t, H), dtype=torch.bfloat16, device=dev) for t in tokens]
        for r, t in enumerate(tokens):
            x, sf, ti, tw = eng.input_views(r)
            x[:t].copy_(xs[r][0]); sf[:t].copy_(xs[r][1]); ti[:t].copy_(idx[r].to(torch.int32)); tw[:t].copy_(ws[r])
        for fused in (True, False):
            eng.forward(ys, tokens, w1s, w2s, fused=fused)
            torch.cuda.synchronize()
            eng.check()
            for r in range(world):
                ok, bad, worst = _mixed_error_ok(ys[r].cpu(), ref[r])
                assert ok, f"rank {r} (fused={fused}): {bad:.4f} of elements off, worst relative error {worst:.4f}"
    finally:
        torch.cuda.synchronize()
        for s in sessions:
            s.close()


def test_fp8_weights_public_api():
    """``mma_type="fp8xfp8"``: e4m3 weights with ue8m0 scales per 32 (routed and shared) through the same fused kernel."""
    from deepep_b200.models.mega_moe import SymmBuffer, fp8_fp4_mega_moe, transform_weights_for_mega_moe

    dev = torch.device("cuda")
    T, H, I, E, K, S = 160, 512, 256, 4, 2, 1
    l1, l2 = O.make_fp8_weights(E, H, I, 21)
    sl1, sl2 = O.make_fp8_weights(S, H, I, 22)
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(5)).bfloat16()
    idx, w = make_routes("random", T, E, K, 1, 9), make_weights(T, K, 4)
    ref = O.mega_moe_reference([O.quantize_mxfp8(x)], [idx], [w], l1, l2, E, sl1, sl2)[0]
    buf = SymmBuffer(None, E, 256, K, H, I, num_shared_experts=S, mma_type="fp8xfp8")
    try:
        w1, w2 = transform_weights_for_mega_moe(l1, l2, device=dev)
        sw1, sw2 = transform_weights_for_mega_moe(sl1, sl2, device=dev)
        assert w1.fp8 and w2.fp8 and w1.packed.shape[1] == 128
        buf.topk_idx[:T].copy_(idx.to(torch.int32)); buf.topk_weights[:T].copy_(w)
        y = torch.zeros((T, H), dtype=torch.bfloat16, device=dev)
        for fused in (True, False):
            y.zero_()
            fp8_fp4_mega_moe(y, w1, w2, buf, sw1, sw2, x=x.to(dev), fused=fused, check=True)
            ok, bad, worst = _mixed_error_ok(y.cpu(), ref)
            assert ok, f"fused={fused}: {bad:.4f} of elements off, worst relative error {worst:.4f}"
        e2m1 = transform_weights_for_mega_moe(*O.make_weights(E, H, I, 3), device=dev)
        with pytest.raises(ValueError, match="mma_type"):
            fp8_fp4_mega_moe(y, e2m1[0], e2m1[1], buf, sw1, sw2)          # e2m1 weights on an fp8xfp8 buffer
    finally:
        buf.destroy()
