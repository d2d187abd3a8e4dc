"""The allocation-free routing-layout entry point, called through its exported C symbol.

It is meant for hosts that must not allocate device memory while running (a serving process whose memory
pool owns the whole GPU, or a C caller without a tensor framework): all scratch lives in a fixed array
inside the library.  The test calls it twice in a row with different inputs -- the scratch array keeps the
first call's contents -- and checks every output against the regular entry point (whose scratch is
allocated through torch).  This file sorts last on purpose, so a failure here cannot hide other tests.
"""
import ctypes

import pytest
import torch

from helpers import make_routes, make_weights

pytestmark = pytest.mark.gpu

MAX_TOKENS = 4096


def _regular(idx, w, E, alignment):
    from deepep_b200.parallel.virtual import VirtualWorld

    T, K = idx.shape
    with VirtualWorld(1, max(T, 1), 64, K, timeout=10.0) as vw:
        plan = vw.engine.notify([idx], [w], E, expand=True, alignment=alignment)[0]
        torch.cuda.synchronize()
        return plan


def _no_alloc(lib, idx, w, E, alignment):
    dev = idx.device
    T, K = idx.shape
    stride = 2 + max(2, min(K, E))
    cap = T * min(K, E) + E * (alignment - 1)
    i32 = dict(dtype=torch.int32, device=dev)
    out = dict(send_slot=torch.full((max(T, 1),), -7, **i32), slot_row=torch.full((max(T, 1), K), -7, **i32),
               stage_meta=torch.zeros((MAX_TOKENS, stride), **i32), chunk_start=torch.zeros((MAX_TOKENS // 64 + 1,), **i32),
               expert_counts=torch.zeros((E,), **i32), expert_offsets=torch.zeros((E + 1,), **i32),
               recv_row_src=torch.full((max(cap, 1),), -7, **i32), recv_w=torch.zeros((max(cap, 1),), dtype=torch.float32, device=dev),
               info=torch.zeros((4 + E,), **i32))
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.deepep_notify_layout_noalloc(p(idx), p(w), T, K, E, alignment, p(out["send_slot"]), p(out["slot_row"]),
                                          p(out["stage_meta"]), p(out["chunk_start"]), p(out["expert_counts"]), p(out["expert_offsets"]),
                                          p(out["recv_row_src"]), p(out["recv_w"]), ctypes.c_longlong(cap), p(out["info"]),
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.deepep_noalloc_last_error().decode()
    torch.cuda.synchronize()
    return out


def test_no_alloc_entry_matches_regular_entry_twice():
    from deepep_b200.ops import native_path

    lib = ctypes.CDLL(str(native_path()))
    lib.deepep_notify_layout_noalloc.restype = ctypes.c_int
    lib.deepep_noalloc_last_error.restype = ctypes.c_char_p
    dev = torch.device("cuda")
    for call, (T, K, E, alignment, mode) in enumerate([(1000, 8, 64, 1, "random"), (333, 4, 16, 8, "invalid")]):
        idx, w = make_routes(mode, T, E, K, 1, seed=call).to(dev), make_weights(T, K, call).to(dev)
        got, plan = _no_alloc(lib, idx, w, E, alignment), _regular(idx, w, E, alignment)
        rows, staged = plan.num_rows, plan.num_staged_rows
        info = got["info"].cpu().tolist()
        assert info[0] == rows and info[1] == staged and info[4:4 + E] == plan.expert_counts_list
        assert torch.equal(got["expert_counts"], plan.expert_counts) and torch.equal(got["expert_offsets"], plan.expert_offsets)
        assert torch.equal(got["send_slot"][:T], plan.send_slot[:T, 0]) and torch.equal(got["slot_row"][:T], plan.slot_row[:T])
        assert torch.equal(got["recv_row_src"][:rows], plan.recv_row_src[:rows])
        assert torch.equal(got["recv_w"][:rows], plan.recv_w[:rows])          # exact: both copy the caller's fp32 weights
        n = plan.stage_meta[:staged, 1:2]
        cols = torch.arange(plan.meta_stride, device=dev).unsqueeze(0)
        used = cols < (2 + n)                                                   # token, n, then n row entries
        assert torch.equal(torch.where(used, got["stage_meta"][:staged], 0), torch.where(used, plan.stage_meta[:staged], 0))
        tiles = -(-T // 64)
        assert torch.equal(got["chunk_start"][:tiles + 1], plan.chunk_start[0, :tiles + 1])


def test_no_alloc_entry_rejects_capacity_without_padding_rows():
    """With an alignment above 1 the padding rows are written too: a capacity that leaves them out is refused up front."""
    from deepep_b200.ops import native_path

    lib = ctypes.CDLL(str(native_path()))
    lib.deepep_notify_layout_noalloc.restype = ctypes.c_int
    lib.deepep_noalloc_last_error.restype = ctypes.c_char_p
    one = ctypes.c_void_p(256)   # never dereferenced: the call is refused before any launch
    T, K, E, alignment = 333, 4, 16, 8
    rc = lib.deepep_notify_layout_noalloc(one, None, T, K, E, alignment, one, one, one, one, one, one, one, None,
                                          ctypes.c_longlong(T * K), one, None)
    assert rc != 0 and b"expert_alignment - 1" in lib.deepep_noalloc_last_error()


def test_no_alloc_entry_rejects_oversize():
    from deepep_b200.ops import native_path

    lib = ctypes.CDLL(str(native_path()))
    lib.deepep_notify_layout_noalloc.restype = ctypes.c_int
    lib.deepep_noalloc_last_error.restype = ctypes.c_char_p
    null = ctypes.c_void_p(0)
    rc = lib.deepep_notify_layout_noalloc(null, null, MAX_TOKENS + 1, 8, 64, 1, null, null, null, null, null, null, null, null,
                                          ctypes.c_longlong(0), null, null)
    assert rc != 0 and b"DEEPEP_NOALLOC_MAX_TOKENS" in lib.deepep_noalloc_last_error()
