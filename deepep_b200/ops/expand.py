"""``expand`` / ``aggregate``: local layout operators of the V1 interface.

``expand`` turns rank-deduplicated dispatch rows (one row per received token carrying up to K local expert ids) into
expert-major rows (one row per (token, slot), sorted by expert, then row, then slot, every expert's block padded to its
capacity with zero rows); ``aggregate`` is the inverse reduction (fp32 sum in slot order, optional per-row weights, an
independent fp32 value channel).  Parity: ``Buffer.expand`` / ``Buffer.aggregate`` of the reference
(``deep_ep/backends/direct/buffer.py:753-918``, ``expand.py:8-40``; kernels ``csrc/direct/kernels/expand/expand.cpp``
and ``aggregate/aggregate.cpp``).  CUDA tensors run the native kernels (``csrc/kernels/expand.cu``); CPU tensors run
the plain restatement below, which is also the oracle of the GPU tests.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple, Union

import torch


class ExpandHandle:
    """Reusable mapping between rank-deduplicated and expert-major rows."""

    __slots__ = ("expert_offsets", "actual_expert_counts", "recv_to_expanded_idx", "num_tokens_per_expert_list",
                 "num_recv_tokens", "num_expanded_tokens", "num_topk", "expert_alignment")

    def __init__(self, expert_offsets, actual_expert_counts, recv_to_expanded_idx, num_tokens_per_expert_list: List[int],
                 num_recv_tokens: int, num_expanded_tokens: int, num_topk: int, expert_alignment: int) -> None:
        self.expert_offsets = expert_offsets
        self.actual_expert_counts = actual_expert_counts
        self.recv_to_expanded_idx = recv_to_expanded_idx
        self.num_tokens_per_expert_list = list(num_tokens_per_expert_list)
        self.num_recv_tokens = int(num_recv_tokens)
        self.num_expanded_tokens = int(num_expanded_tokens)
        self.num_topk = int(num_topk)
        self.expert_alignment = int(expert_alignment)


def validate_expand_counts(counts: Sequence[int], expert_alignment: int) -> List[int]:
    if not isinstance(expert_alignment, int) or isinstance(expert_alignment, bool):
        raise TypeError("expert_alignment must be an integer")
    if expert_alignment <= 0:
        raise ValueError("expert_alignment must be positive")
    if not isinstance(counts, (list, tuple)) or not counts:
        raise TypeError("num_tokens_per_expert must be a non-empty list")
    for c in counts:
        if not isinstance(c, int) or isinstance(c, bool):
            raise TypeError("expert token counts must be integers")
        if c < 0:
            raise ValueError("expert token counts must be nonnegative")
        if c % expert_alignment:
            raise ValueError("expert token counts must be aligned to expert_alignment")
    return list(counts)


# ------------------------------------------------------------------------------------------------ restatement
def reference_mapping(topk_idx: torch.Tensor, capacities: Sequence[int]) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(expert_offsets int32 [L + 1], actual counts int32 [L], mapping int32 [R, K]) in (expert, row, slot) order."""
    L = len(capacities)
    offsets = torch.zeros(L + 1, dtype=torch.int32)
    offsets[1:] = torch.tensor(list(capacities), dtype=torch.int64).cumsum(0).to(torch.int32)
    idx = topk_idx.cpu()
    mapping = torch.full(idx.shape, -1, dtype=torch.int32)
    counts = [0] * L
    for r in range(idx.shape[0]):
        seen = set()
        for k in range(idx.shape[1]):
            e = int(idx[r, k])
            if 0 <= e < L and e not in seen:
                seen.add(e)
                if counts[e] < capacities[e]:
                    mapping[r, k] = int(offsets[e]) + counts[e]
                counts[e] += 1
    return offsets, torch.tensor(counts, dtype=torch.int32), mapping


def _expand_cpu(x, x_sf, topk_w, mapping, total):
    out = torch.zeros((total, x.shape[1]), dtype=x.dtype)
    out_sf = torch.zeros((total, x_sf.shape[1]), dtype=torch.float32) if x_sf is not None else None
    out_w = torch.zeros((total,), dtype=torch.float32) if topk_w is not None else None
    rows, slots = (mapping >= 0).nonzero(as_tuple=True)
    dst = mapping[rows, slots].long()
    if x.dtype == torch.float8_e4m3fn:
        out.view(torch.uint8)[dst] = x.view(torch.uint8)[rows]
    else:
        out[dst] = x[rows]
    if out_sf is not None:
        out_sf[dst] = x_sf[rows]
    if out_w is not None:
        out_w[dst] = topk_w[rows, slots]
    return out, out_sf, out_w


def _aggregate_cpu(x, row_w, values, mapping):
    R, K = mapping.shape
    acc = torch.zeros((R, x.shape[1]), dtype=torch.float32)
    out_values = torch.zeros((R, K), dtype=torch.float32) if values is not None else None
    for k in range(K):                       # slot order fixes the fp32 summation order
        d = mapping[:, k].long()
        ok = d >= 0
        rows = x[d.clamp(min=0)].float()
        if row_w is not None:
            rows = rows * row_w[d.clamp(min=0)].unsqueeze(1)
        acc = torch.where(ok.unsqueeze(1), acc + rows, acc)
        if out_values is not None:
            out_values[:, k] = torch.where(ok, values[d.clamp(min=0)], torch.zeros(()))
    return acc.to(x.dtype), out_values


# ------------------------------------------------------------------------------------------------ operators
def _blocks(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count * 2


def expand(x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]], recv_topk_idx: Optional[torch.Tensor] = None,
           topk_weights: Optional[torch.Tensor] = None, num_tokens_per_expert: Optional[List[int]] = None,
           expert_alignment: Optional[int] = None, handle: Optional[ExpandHandle] = None, stream=None):
    """Returns ``(expanded_x | (expanded_x, expanded_scales), expanded_topk_weights, handle)``.

    Fresh call: ``recv_topk_idx`` ``[R, K]`` (local expert ids, anything outside ``[0, L)`` is an empty slot) and
    ``num_tokens_per_expert`` (every expert's capacity, a multiple of ``expert_alignment``) are required.  An expert
    that receives more rows than its capacity raises ``ValueError`` (after a device synchronisation).  Cached call:
    pass the ``handle`` of an earlier call and neither of the two.
    """
    data, scales = (x if isinstance(x, (tuple, list)) else (x, None))
    if data.dim() != 2 or not data.is_contiguous() or (data.shape[1] * data.element_size()) % 16:
        raise ValueError("x must be a contiguous [num_recv_tokens, hidden] tensor whose rows are a multiple of 16 bytes")
    if scales is not None and (scales.dim() != 2 or scales.shape[0] != data.shape[0] or scales.dtype != torch.float32 or not scales.is_contiguous()):
        raise ValueError("scales must be a contiguous fp32 [num_recv_tokens, num_scales] tensor")
    R = data.shape[0]
    if handle is None:
        if recv_topk_idx is None:
            raise ValueError("recv_topk_idx is required for non-cached expand")
        if num_tokens_per_expert is None:
            raise ValueError("num_tokens_per_expert is required for non-cached expand")
        expert_alignment = 1 if expert_alignment is None else expert_alignment
        caps = validate_expand_counts(num_tokens_per_expert, expert_alignment)
        if recv_topk_idx.dim() != 2 or recv_topk_idx.shape[0] != R or recv_topk_idx.dtype != torch.int64 or not recv_topk_idx.is_contiguous():
            raise ValueError("recv_topk_idx must be a contiguous int64 [num_recv_tokens, num_topk] tensor")
        K, total = recv_topk_idx.shape[1], sum(caps)
    else:
        if not isinstance(handle, ExpandHandle):
            raise TypeError("handle must be an ExpandHandle")
        if R != handle.num_recv_tokens:
            raise ValueError("cached expand x must match the handle num_recv_tokens")
        if recv_topk_idx is not None:
            raise ValueError("cached expand requires recv_topk_idx=None")
        if num_tokens_per_expert is not None:
            raise ValueError("cached expand requires num_tokens_per_expert=None")
        if expert_alignment is not None and expert_alignment != handle.expert_alignment:
            raise ValueError("cached expand expert_alignment must match the handle")
        caps, K, total, expert_alignment = handle.num_tokens_per_expert_list, handle.num_topk, handle.num_expanded_tokens, handle.expert_alignment
    if topk_weights is not None and (tuple(topk_weights.shape) != (R, K) or topk_weights.dtype != torch.float32 or not topk_weights.is_contiguous()):
        raise ValueError("topk_weights must be a contiguous fp32 [num_recv_tokens, num_topk] tensor")
    L = len(caps)

    if data.device.type != "cuda":
        if handle is None:
            offsets, actual, mapping = reference_mapping(recv_topk_idx, caps)
            if bool((actual > torch.tensor(caps, dtype=torch.int32)).any()):
                raise ValueError("an expert received more rows than its capacity in num_tokens_per_expert")
            handle = ExpandHandle(offsets, actual, mapping, caps, R, total, K, expert_alignment)
        out, out_sf, out_w = _expand_cpu(data, scales, topk_weights, handle.recv_to_expanded_idx, total)
        return ((out, out_sf) if scales is not None else out), out_w, handle

    from . import require_native

    C = require_native("expand")
    dev = data.device
    stream = torch.cuda.current_stream(dev) if stream is None else stream
    i32 = dict(dtype=torch.int32, device=dev)
    out = torch.empty((total, data.shape[1]), dtype=data.dtype, device=dev)
    out_sf = torch.empty((total, scales.shape[1]), dtype=torch.float32, device=dev) if scales is not None else None
    out_w = torch.empty((total,), dtype=torch.float32, device=dev) if topk_weights is not None else None
    err = torch.zeros((1,), **i32)
    if handle is None:
        offsets = torch.zeros((L + 1,), dtype=torch.int32)
        offsets[1:] = torch.tensor(caps, dtype=torch.int64).cumsum(0).to(torch.int32)
        offsets = offsets.to(dev)
        actual = torch.empty((L,), **i32)
        mapping = torch.empty((R, K), **i32)
        tiles = -(-R // C.expand_tile)
        tile_counts = torch.empty((max(tiles, 1) * L,), **i32)
    else:
        offsets, actual, mapping, tile_counts = handle.expert_offsets, handle.actual_expert_counts, handle.recv_to_expanded_idx, None
    C.expand(dict(x=data.data_ptr() if R else None, x_sf=scales.data_ptr() if scales is not None and R else (scales.data_ptr() if scales is not None else None),
                  topk_idx=recv_topk_idx.data_ptr() if recv_topk_idx is not None and R else None,
                  topk_w=topk_weights.data_ptr() if topk_weights is not None and R else None,
                  out=out.data_ptr() if total else None, out_sf=out_sf.data_ptr() if out_sf is not None else None,
                  out_w=out_w.data_ptr() if out_w is not None else None, expert_offsets=offsets.data_ptr(),
                  actual_counts=actual.data_ptr(), mapping=mapping.data_ptr() if R else None,
                  tile_counts=tile_counts.data_ptr() if tile_counts is not None else None, err=err.data_ptr(), rows=R, topk=K,
                  experts=L, expanded_rows=total, row_bytes=data.shape[1] * data.element_size(),
                  num_sf=scales.shape[1] if scales is not None else 0, cached=int(handle is not None)),
             _blocks(dev), stream.cuda_stream)
    if handle is None:
        if int(err.item()):
            raise ValueError("an expert received more rows than its capacity in num_tokens_per_expert")
        handle = ExpandHandle(offsets, actual, mapping, caps, R, total, K, expert_alignment)
    return ((out, out_sf) if scales is not None else out), out_w, handle


def aggregate(x: torch.Tensor, handle: ExpandHandle, topk_weights: Optional[torch.Tensor] = None,
              expanded_values: Optional[torch.Tensor] = None, stream=None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Returns ``(aggregated_x [R, H], aggregated_values [R, K] | None)``: ``aggregated_x[r] = sum_k (w *) x[map[r, k]]``
    (fp32, slot order); ``topk_weights`` ``[N]`` multiplies every expanded row, ``expanded_values`` ``[N]`` is an
    independent fp32 channel returned per (row, slot)."""
    if not isinstance(handle, ExpandHandle):
        raise TypeError("handle must be an ExpandHandle")
    if x.dim() != 2 or x.shape[0] != handle.num_expanded_tokens:
        raise ValueError("aggregate x must match the handle num_expanded_tokens")
    if x.dtype not in (torch.bfloat16, torch.float16) or not x.is_contiguous() or x.shape[1] % 8:
        raise ValueError("x must be a contiguous bf16 or fp16 tensor whose hidden size is a multiple of 8")
    N, R, K = x.shape[0], handle.num_recv_tokens, handle.num_topk
    for name, t in (("topk_weights", topk_weights), ("expanded_values", expanded_values)):
        if t is not None and (tuple(t.shape) != (N,) or t.dtype != torch.float32 or not t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous fp32 [num_expanded_tokens] tensor")
    if x.device.type != "cuda":
        return _aggregate_cpu(x, topk_weights, expanded_values, handle.recv_to_expanded_idx)
    from . import require_native

    C = require_native("aggregate")
    dev = x.device
    stream = torch.cuda.current_stream(dev) if stream is None else stream
    out = torch.empty((R, x.shape[1]), dtype=x.dtype, device=dev)
    out_values = torch.empty((R, K), dtype=torch.float32, device=dev) if expanded_values is not None else None
    C.aggregate(dict(x=x.data_ptr() if N else None, row_w=topk_weights.data_ptr() if topk_weights is not None and N else None,
                     values=expanded_values.data_ptr() if expanded_values is not None and N else None,
                     mapping=handle.recv_to_expanded_idx.data_ptr() if R else None, out=out.data_ptr() if R else None,
                     out_values=out_values.data_ptr() if out_values is not None and R else None, rows=R, topk=K,
                     hidden=x.shape[1], expanded_rows=N, is_half=int(x.dtype == torch.float16)), _blocks(dev), stream.cuda_stream)
    return out, out_values


__all__ = ["ExpandHandle", "aggregate", "expand", "reference_mapping", "validate_expand_counts"]
