"""CPU oracle of the fused MoE forward (MXFP8 activations x MXFP4 weights), in torch.

Same math as the reference's NumPy oracle (``experiments/megamoe/python/deep_ep_experimental/megamoe/
reference.py:17-110``): per-32 block scales ``2^(floor(log2(amax)) - 8)`` with e4m3 saturation,
e2m1 weights (low nibble = even element) times ue8m0 scales, ``bf16(x @ W1^T)`` -> split gate/up ->
``bf16(silu(gate) * up)`` -> MXFP8 requantisation -> ``bf16(. @ W2^T)``, and the route weight applied after
the second GEMM while summing the top-k contributions in fp32.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

FP4_VALUES = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float32)


def bf16(x: torch.Tensor) -> torch.Tensor:
    return x.float().bfloat16().float()


def quantize_mxfp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[..., K] -> (e4m3 codes [..., K], ue8m0 exponents uint8 [..., K / 32])."""
    x = bf16(x)
    assert x.shape[-1] % 32 == 0
    blocks = x.reshape(*x.shape[:-1], x.shape[-1] // 32, 32)
    amax = blocks.abs().amax(dim=-1)
    exponent = torch.clamp(torch.floor(torch.log2(torch.clamp(amax, min=2.0 ** -119))) - 8, min=-127)
    scaled = (blocks / torch.exp2(exponent).unsqueeze(-1)).clamp(-448, 448)
    return scaled.reshape(x.shape).to(torch.float8_e4m3fn), (exponent + 127).to(torch.uint8)


def dequantize_mxfp8(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    scale = torch.exp2(scales.float() - 127)
    return codes.float() * scale.repeat_interleave(32, dim=-1)


def unpack_fp4(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """packed uint8 [..., K / 2] (low nibble first), scales uint8 [..., K / 32] -> fp32 [..., K]."""
    lo, hi = FP4_VALUES[(packed & 15).long()], FP4_VALUES[(packed >> 4).long()]
    values = torch.stack((lo, hi), dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    return values * torch.exp2(scales.reshape(*values.shape[:-1], -1).float() - 127).repeat_interleave(32, dim=-1)


def unpack_weights(w: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Weights of either kind -> fp32: packed e2m1 pairs (uint8 [..., K / 2]) or e4m3 ([..., K]), ue8m0 scales per 32."""
    if w.dtype == torch.float8_e4m3fn:
        return dequantize_mxfp8(w, scales.reshape(*w.shape[:-1], -1))
    return unpack_fp4(w, scales)


def make_fp8_weights(experts: int, hidden: int, intermediate: int, seed: int):
    """Random e4m3 weights with ue8m0 scales per 32 (A8W8): ((w1 [E, 2I, H], w1_sf [E, 2I, H / 32]), (w2, w2_sf))."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for n, k in ((2 * intermediate, hidden), (hidden, intermediate)):
        w = torch.randn((experts, n, k), generator=g) * (k ** -0.5)
        out.append(quantize_mxfp8(w))
    return tuple(out)


def tile_rows(rows: torch.Tensor, width: int) -> torch.Tensor:
    """[rows, bytes per row] uint8 -> every (128-row, `width`-byte) block contiguous (width = bytes of 128 K-values)."""
    n, kb = rows.shape
    assert n % 128 == 0 and kb % width == 0
    return rows.view(n // 128, 128, kb // width, width).permute(0, 2, 1, 3).contiguous().view(-1, width)


def make_weights(experts: int, hidden: int, intermediate: int, seed: int):
    """Random packed e2m1 weights with non-uniform ue8m0 scales: ((w1, w1_sf), (w2, w2_sf))."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for n, k in ((2 * intermediate, hidden), (hidden, intermediate)):
        packed = torch.randint(0, 256, (experts, n, k // 2), generator=g, dtype=torch.uint8)
        exponent = int(torch.floor(-0.5 * torch.log2(torch.tensor(float(k))))) - 2
        scales = torch.randint(127 + exponent - 1, 127 + exponent + 2, (experts, n, k // 32), generator=g, dtype=torch.uint8)
        out.append((packed, scales))
    return tuple(out)


def expert_forward(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    first = bf16(x @ w1.t())
    gate, up = first.chunk(2, dim=-1)
    activated = bf16(gate / (1 + torch.exp(torch.clamp(-gate, -80, 80))) * up)
    q = dequantize_mxfp8(*quantize_mxfp8(activated))
    return bf16(q @ w2.t())


def mega_moe_reference(xs: Sequence[Tuple[torch.Tensor, torch.Tensor]], topk_idx: Sequence[torch.Tensor],
                       topk_w: Sequence[torch.Tensor], l1, l2, num_experts: int, shared_l1=None, shared_l2=None) -> List[torch.Tensor]:
    """All-rank forward.  xs[r] = (e4m3 [T, H], ue8m0 [T, H / 32]); l1/l2 = (packed, scales) for all experts.
    ``shared_l1`` / ``shared_l2``: weights of the shared experts (the same on every rank); every token passes through
    each of them with weight one, after its routed experts (``golden.py:160-165`` of the reference)."""
    w1 = unpack_weights(*l1)
    w2 = unpack_weights(*l2)
    s1 = None if shared_l1 is None else unpack_weights(*shared_l1)
    s2 = None if shared_l2 is None else unpack_weights(*shared_l2)
    outs = []
    for (codes, sf), idx, w in zip(xs, topk_idx, topk_w):
        x = dequantize_mxfp8(codes, sf)
        y = torch.zeros_like(x)
        for k in range(idx.shape[1]):          # slot order fixes the fp32 summation order
            for e in idx[:, k].unique().tolist():
                if e < 0 or e >= num_experts:
                    continue
                tok = (idx[:, k] == e).nonzero(as_tuple=True)[0]
                y[tok] += w[tok, k].float().unsqueeze(1) * expert_forward(x[tok], w1[e], w2[e])
        if s1 is not None and x.shape[0]:
            for e in range(s1.shape[0]):
                y += expert_forward(x, s1[e], s2[e])
        outs.append(y.bfloat16())
    return outs


def to_sf_chunks(sf: torch.Tensor) -> torch.Tensor:
    """[rows, K / 32] ue8m0 -> the 512-byte chunk image the tensor cores read (rows and K / 32 padded to 128 / 4)."""
    rows, kb = sf.shape
    rp, kp = -(-rows // 128) * 128, -(-kb // 4) * 4
    full = torch.zeros((rp, kp), dtype=torch.uint8, device=sf.device)
    full[:rows, :kb] = sf
    v = full.view(rp // 128, 4, 32, kp // 4, 4)          # [row block, row / 32, row % 32, K block, k / 32 % 4]
    return v.permute(0, 3, 2, 1, 4).contiguous().view(-1)


def tile_fp4_rows(packed: torch.Tensor) -> torch.Tensor:
    """[rows, K / 2] packed e2m1 -> [(rows / 128) * (K / 128) * 128, 64]: every (128-row, 128-K) block becomes 8 KB of
    contiguous memory, so one tile load of the GEMM reads one contiguous block instead of 128 strided 64-byte pieces."""
    return tile_rows(packed, 64)


__all__ = ["tile_fp4_rows", "tile_rows", "unpack_weights", "make_fp8_weights", "bf16", "dequantize_mxfp8", "expert_forward", "make_weights", "mega_moe_reference", "quantize_mxfp8",
           "to_sf_chunks", "unpack_fp4"]
