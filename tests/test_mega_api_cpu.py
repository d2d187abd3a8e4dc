"""Host side of the fused MoE API without a GPU: the input loader of ``SymmBuffer`` (ue8m0 codes from power-of-two fp32
block scales), the argument rules of ``fp8_fp4_mega_moe`` in the order the reference states them
(``experiments/megamoe/python/deep_ep_experimental/megamoe/api.py:520-567``), shared-expert weight joining and the
statistics update.  The buffer object is assembled by hand around a recording engine; no kernel runs.
"""
import pytest
import torch

from deepep_b200.models import mega_moe as MM
from deepep_b200.oracle import megamoe as O
from deepep_b200.utils.math import per_token_cast_to_fp8

H, I, K, E, M = 256, 128, 2, 4, 16


class RecordingEngine:
    def __init__(self):
        self.calls, self.sm_count = [], 4
        self.scratch = [dict(expert_rows=torch.tensor([3, 0, 5, 1, 9], dtype=torch.int32))]
        self.checked = 0

    def forward(self, ys, tokens, l1, l2, fused=True, x_bf16=None, timer=None):
        self.calls.append(dict(ys=ys, tokens=tokens, l1=l1, l2=l2, fused=fused, x_bf16=x_bf16, timer=timer))

    def check(self):
        self.checked += 1


def make_buffer(shared=0, mma_type="fp8xfp4", world=1):
    sym = object.__new__(MM.SymmBuffer)
    sym.hidden, sym.intermediate_hidden, sym.num_topk, sym.num_experts = H, I, K, E
    sym.num_max_tokens_per_rank, sym.num_shared_experts, sym.mma_type, sym.world_size = M, shared, mma_type, world
    sym.device = torch.device("cpu")
    sym.x = torch.zeros((M, H), dtype=torch.float8_e4m3fn)
    sym.x_sf = torch.zeros((M, H // 32), dtype=torch.uint8)
    sym.topk_idx = torch.full((M, K), -1, dtype=torch.int32)
    sym.topk_weights = torch.zeros((M, K), dtype=torch.float32)
    sym.engine, sym._joined, sym.batch_size = RecordingEngine(), {}, 0
    return sym


def weights(experts=E, seed=0):
    return MM.transform_weights_for_mega_moe(*O.make_weights(experts, H, I, seed))


def test_load_inputs_converts_power_of_two_block_scales():
    sym = make_buffer()
    x = torch.randn((5, H), generator=torch.Generator().manual_seed(2)) * 4
    q, scale = per_token_cast_to_fp8(x, use_ue8m0=True)                       # fp32 [5, H / 128], powers of two
    idx = torch.tensor([[0, 1], [2, 3], [1, -1], [0, 3], [2, 1]])
    w = torch.rand((5, K))
    assert sym.load_inputs(q, scale, idx, w) is sym and sym.batch_size == 5
    # every 128-block scale serves its four 32-value blocks; decoding the codes gives the input scales back exactly
    decoded = torch.exp2(sym.x_sf[:5].float() - 127)
    assert torch.equal(decoded, scale.repeat_interleave(4, dim=1))
    assert torch.equal(sym.x[:5].view(torch.uint8), q.view(torch.uint8))
    assert sym.topk_idx[:5].tolist() == idx.tolist() and torch.equal(sym.topk_weights[:5], w)
    assert torch.equal(O.dequantize_mxfp8(sym.x[:5], sym.x_sf[:5]), (q.float().view(5, -1, 128) * scale.unsqueeze(2)).view(5, H))
    # ue8m0 codes are taken as they are
    codes, sf = O.quantize_mxfp8(x)
    sym.load_inputs(codes, sf, idx, w)
    assert torch.equal(sym.x_sf[:5], sf)
    # scales that ue8m0 cannot carry exactly are refused, as are wrong shapes and oversized batches
    with pytest.raises(ValueError, match="powers of two"):
        sym.load_inputs(q, scale * 1.5, idx, w)
    with pytest.raises(ValueError, match="x_sf must be"):
        sym.load_inputs(q, scale[:, :1], idx, w)
    with pytest.raises(ValueError, match="e4m3"):
        sym.load_inputs(q.float(), scale, idx, w)
    big = torch.zeros((M + 1, H), dtype=torch.float8_e4m3fn)
    with pytest.raises(ValueError, match="batch"):
        sym.load_inputs(big, torch.ones((M + 1, H // 128)), idx, w)
    with pytest.raises(ValueError, match="batch size"):
        sym.prepare(M + 1)
    sym.validate_inputs(5, x=torch.zeros((5, H), dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="x override"):
        sym.validate_inputs(5, x=torch.zeros((5, H)))
    with pytest.raises(ValueError, match="batch size"):
        sym.validate_inputs(0)
    sym.topk_idx[0, 0] = E
    with pytest.raises(ValueError, match="outside"):
        sym.validate_inputs(5)
    sym.topk_idx[0, 0] = 0
    sym.topk_weights[1, 1] = float("nan")
    with pytest.raises(ValueError, match="finite"):
        sym.validate_inputs(5)


def test_forward_argument_rules_and_what_reaches_the_engine():
    sym, (l1, l2) = make_buffer(), weights()
    y = torch.zeros((6, H), dtype=torch.bfloat16)
    stats = torch.tensor([10, 10, 10, 10], dtype=torch.int32)
    assert MM.fp8_fp4_mega_moe(y, l1, l2, sym, cumulative_local_expert_recv_stats=stats) is None
    call = sym.engine.calls[-1]
    assert call["ys"][0] is y and call["tokens"] == [6] and call["l1"][0] is l1 and call["l2"][0] is l2
    assert call["fused"] is True and call["x_bf16"] is None and call["timer"] is None
    assert stats.tolist() == [13, 10, 15, 11]                                  # the routed experts' rows, not the fifth entry
    xb = torch.zeros((6, H), dtype=torch.bfloat16)
    MM.fp8_fp4_mega_moe(y, l1, l2, sym, x=xb, fused=False)
    assert sym.engine.calls[-1]["x_bf16"][0] is xb and sym.engine.calls[-1]["fused"] is False and sym.engine.checked == 0
    for kwargs, kind, message in (
            (dict(recipe=(1, 1, 128)), NotImplementedError, "recipe"),
            (dict(activation="gelu"), NotImplementedError, "SwiGLU"),
            (dict(activation_clamp=7.0), NotImplementedError, "SwiGLU"),
            (dict(fast_math=False), NotImplementedError, "SwiGLU"),
            (dict(shared_l1_weights=l1), ValueError, "both shared"),
            (dict(shared_l1_weights=l1, shared_l2_weights=l2), ValueError, "num_shared_experts"),
            (dict(x=xb.float()), ValueError, "x override"),
            (dict(cumulative_local_expert_recv_stats=stats.long()), ValueError, "int32"),
            (dict(timer=torch.zeros((4, 8), dtype=torch.int32)), ValueError, "allocate_timer"),
            (dict(timer=torch.zeros((4, 8), dtype=torch.int64), fused=False), ValueError, "fused")):
        with pytest.raises(kind, match=message):
            MM.fp8_fp4_mega_moe(y, l1, l2, sym, **kwargs)
    with pytest.raises(TypeError, match="SymmBuffer"):
        MM.fp8_fp4_mega_moe(y, l1, l2, object())
    with pytest.raises(TypeError, match="transform_weights"):
        MM.fp8_fp4_mega_moe(y, (None, None), l2, sym)
    with pytest.raises(ValueError, match="bf16"):
        MM.fp8_fp4_mega_moe(y.float(), l1, l2, sym)
    with pytest.raises(ValueError, match="non-empty"):
        MM.fp8_fp4_mega_moe(y[:0], l1, l2, sym)
    with pytest.raises(ValueError, match="experts"):
        MM.fp8_fp4_mega_moe(y, *weights(experts=2), sym)
    with pytest.raises(ValueError, match="other kind"):
        MM.fp8_fp4_mega_moe(y, l1, l2, make_buffer(mma_type="fp8xfp8"))


def test_shared_experts_are_joined_once_per_weight_set():
    sym, (l1, l2), (s1, s2) = make_buffer(shared=1), weights(), weights(experts=1, seed=9)
    y = torch.zeros((4, H), dtype=torch.bfloat16)
    MM.fp8_fp4_mega_moe(y, l1, l2, sym, s1, s2)
    first = sym.engine.calls[-1]
    j1, j2 = first["l1"][0], first["l2"][0]
    assert j1.experts == E + 1 and j2.experts == E + 1 and (j1.n, j1.k, j2.n, j2.k) == (2 * I, H, H, I)
    assert torch.equal(j1.packed[:l1.packed.shape[0]], l1.packed) and torch.equal(j1.packed[l1.packed.shape[0]:], s1.packed)
    assert torch.equal(j2.sf_chunks, torch.cat([l2.sf_chunks, s2.sf_chunks]))
    MM.fp8_fp4_mega_moe(y, l1, l2, sym, s1, s2)
    assert sym.engine.calls[-1]["l1"][0] is j1 and sym.engine.calls[-1]["l2"][0] is j2      # joined once, reused
    f1, f2 = MM.transform_weights_for_mega_moe(*O.make_fp8_weights(1, H, I, 3))
    with pytest.raises(ValueError, match="weight type"):
        sym.joined_weights(l1, f1)
    with pytest.raises(ValueError, match="num_shared_experts"):
        MM.fp8_fp4_mega_moe(y, l1, l2, sym)


def test_weight_transform_shapes_and_rules():
    (w1, w1_sf), (w2, w2_sf) = O.make_weights(E, H, I, 0)
    l1, l2 = MM.transform_weights_for_mega_moe((w1, w1_sf), (w2, w2_sf))
    assert (l1.experts, l1.n, l1.k, l1.fp8) == (E, 2 * I, H, False) and (l2.experts, l2.n, l2.k) == (E, H, I)
    assert l1.packed.dtype == torch.uint8 and l1.packed.numel() == w1.numel() and l2.packed.numel() == w2.numel()
    assert l1.sf_chunks.numel() >= w1_sf.numel() and l1.sf_chunks.numel() % 512 == 0
    (f1, f1_sf), (f2, f2_sf) = O.make_fp8_weights(E, H, I, 1)
    g1, g2 = MM.transform_weights_for_mega_moe((f1, f1_sf), (f2, f2_sf))
    assert g1.fp8 and g2.fp8 and g1.packed.numel() == f1.numel() and (g1.k, g2.k) == (H, I)
    with pytest.raises(ValueError, match="same kind"):
        MM.transform_weights_for_mega_moe((f1, f1_sf), (w2, w2_sf))
    # the reference documents the scales as [L, N, K / 64, 2]: the same bytes, accepted as they are
    r1, r2 = MM.transform_weights_for_mega_moe((w1, w1_sf.view(E, 2 * I, H // 64, 2)), (w2, w2_sf.view(E, H, I // 64, 2)), shared=True)
    assert torch.equal(r1.sf_chunks, l1.sf_chunks) and torch.equal(r2.sf_chunks, l2.sf_chunks) and torch.equal(r1.packed, l1.packed)
    with pytest.raises(NotImplementedError, match="SwiGLU"):
        MM.transform_weights_for_mega_moe((w1, w1_sf), (w2, w2_sf), "gelu")


def test_kernel_failure_report_names_the_wait():
    """``MegaEngine.check`` turns the kernel's error word (which wait ran out) into a message; zero means no failure."""
    eng = object.__new__(MM.MegaEngine)
    eng.scratch = [dict(err=torch.zeros(1, dtype=torch.int32)), dict(err=torch.zeros(1, dtype=torch.int32))]
    eng.check()
    eng.scratch[1]["err"][0] = 8
    with pytest.raises(RuntimeError, match="local rank 1: it was waiting for operands arriving in a stage"):
        eng.check()
    eng.scratch[1]["err"][0] = 77
    with pytest.raises(RuntimeError, match="site 77"):
        eng.check()
    assert set(MM.MegaEngine.WAIT_SITES) == set(range(1, 11))
