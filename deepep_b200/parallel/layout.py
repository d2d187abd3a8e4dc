"""Workspace sizing shared by host code and tests.

Parity: ``deep_ep/backends/mesh_clos/_elastic_layout.py`` of the reference
(``WORLD_SIZES`` :5, ``validate_hidden`` :8-19, ``elastic_size_hint``
:164-173).  The region list differs because the transport differs: a routing
gather area, a dispatch staging area (one row per source token and
destination rank), a combine partial area (one row per token and expert
rank), the returned-weight area, the completion flags of dispatch (one per rank
and pair of source tokens) and of combine (one per rank and block of four
staged rows), and the low-latency region.
"""
from __future__ import annotations

WORLD_SIZES = (1, 2, 4, 8)
MAX_TOKENS = 16384
MAX_TOPK = 16
MAX_HIDDEN = 8192
LL_MAX_TOKENS = 256
LL_SIZE_HINT = 8 << 30
ALIGN = 2 << 20
CONTROL_BYTES = 64 << 10
GROUP_TOKENS = 2           # source tokens per completion flag of the high-throughput dispatch (kGroupTokens in common.cuh)
LL_PARTS = 4               # column parts of a low-latency row, each with its own flag (kLLParts in ll_api.h)
ROW_BLOCK = 4              # staged rows per completion flag of the high-throughput combine (kRowBlock in common.cuh)


def align_up(value: int, alignment: int) -> int:
    return -(-value // alignment) * alignment


def validate_hidden(hidden: int, fp8: bool = False) -> None:
    if not 8 <= hidden <= MAX_HIDDEN:
        raise ValueError(f"hidden must be in [8, {MAX_HIDDEN}]")
    if hidden % 8:
        raise ValueError("hidden must be a multiple of 8 (16-byte rows)")
    if fp8 and hidden % 128:
        raise ValueError("fp8 dispatch needs hidden % 128 == 0 (one scale per 128 values)")


def ll_region_bytes(world: int, max_tokens: int, hidden: int, topk: int) -> int:
    """Bytes of the low-latency region (two banks); 0 when the buffer is too large for that path.

    Mirror of ``make_ll_layout`` in ``csrc/kernels/ll_api.h``: routing gather tables, one flag per column part of a
    row, one staging slot per (source rank, token), one return slot per (token, top-k slot).
    """
    if max_tokens > LL_MAX_TOKENS or max_tokens <= 0:
        return 0
    msg = align_up(hidden * 2, 128)
    at = 0
    for size in (world * 16, world * max_tokens * topk * 4, world * max_tokens * topk * 4, world * 8,
                 world * max_tokens * LL_PARTS * 8, world * max_tokens * msg, max_tokens * topk * LL_PARTS * 8,
                 max_tokens * topk * hidden * 2):
        at = align_up(at + size, 1024)
    return 2 * at


def workspace_bytes(world: int, max_tokens: int, hidden: int, topk: int, ll_bytes: int = 0, mega_bytes: int = 0,
                    partial_tokens: int = 0) -> int:
    """Python mirror of the native ``make_layout`` (checked against it in the tests).  ``partial_tokens``: tokens whose
    combine partials are held at a time (0 = all of them)."""
    window = partial_tokens or max_tokens
    at = CONTROL_BYTES
    stage_row = align_up(hidden * 2, 128)
    groups, row_blocks = -(-max_tokens // GROUP_TOKENS), -(-max_tokens // ROW_BLOCK)
    for size in (world * 4 * 4, world * max_tokens * topk * 4, world * max_tokens * topk * 4,
                 world * max_tokens * stage_row, window * world * hidden * 2, max_tokens * topk * 4,
                 world * groups * 8, world * row_blocks * 8, ll_bytes, mega_bytes):
        at = align_up(at + size, 1024)
    return align_up(at, ALIGN)


def elastic_size_hint(world: int, max_tokens: int, hidden: int, topk: int) -> int:
    if world not in WORLD_SIZES:
        raise ValueError(f"world size must be one of {WORLD_SIZES}")
    if not 0 < max_tokens <= MAX_TOKENS:
        raise ValueError(f"num_max_tokens_per_rank must be in [1, {MAX_TOKENS}]")
    if not 0 < topk <= MAX_TOPK:
        raise ValueError(f"num_topk must be in [1, {MAX_TOPK}]")
    validate_hidden(hidden)
    return workspace_bytes(world, max_tokens, hidden, topk, ll_region_bytes(world, max_tokens, hidden, topk))


def combine_window(world: int, max_tokens: int, hidden: int, topk: int, capacity: int) -> int:
    """Capacity fallback of the combine (parity: ``deep_ep/buffers/_combine_reuse.py:8-34`` of the reference): the largest
    number of tokens whose partials fit a workspace of ``capacity`` bytes, found by bisection; 0 when all tokens fit.
    The other regions (routing tables, dispatch staging, flags, low-latency region) are not windowed: a capacity that
    cannot hold them plus one token's partials is an error."""
    ll = ll_region_bytes(world, max_tokens, hidden, topk)
    if workspace_bytes(world, max_tokens, hidden, topk, ll) <= capacity:
        return 0
    if workspace_bytes(world, max_tokens, hidden, topk, ll, 0, 1) > capacity:
        raise ValueError("num_bytes cannot hold the fixed regions of the workspace and one token's combine partials")
    low, high = 1, max_tokens
    while low < high:
        middle = (low + high + 1) // 2
        if workspace_bytes(world, max_tokens, hidden, topk, ll, 0, middle) <= capacity:
            low = middle
        else:
            high = middle - 1
    return low
