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


def _case(world, tokens, H, I, E, K, seed=0, interleave=None):
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
