"""All-to-all-v fused with a bf16 grouped matmul: ``alltoallv_gmm`` and ``gmm_alltoallv``.

Public API (parity: ``experiments/ep_gmm_fused/python/deep_ep_experimental/ep_gmm_fused/ops.py:182-369`` and
``runtime.py`` of the reference):

* ``init_group(...)`` / ``destroy_group()`` / ``get_config()`` -- the collective set-up of the symmetric workspace
  (the reference's ``init_udma_group`` / ``destroy_udma_group`` / ``get_udma_config``; those names are kept as aliases).
* ``alltoallv_gmm(x, weight, local_tokens_per_expert, global_tokens_per_local_expert, ep_size=, expert_num=, ...)``:
  ``x`` ``[sum(local), k]`` bf16 is sorted by global expert; every row travels to the rank of its expert and is
  multiplied by that expert's ``weight[l]`` (``[k, n]``).  Output ``[received_rows, n]`` ordered by local expert first
  and source rank second; ``output_all_to_allv=True`` also returns the gathered activations.
* ``gmm_alltoallv(x, weight, local_tokens_per_expert, global_tokens_per_local_expert, ep_size=, expert_num=, ...)``:
  ``x`` ``[sum(global), k]`` grouped by (local expert, source rank); the products travel back to the ranks the rows
  came from.  Output ``[sum(local), n]`` in the caller's expert-sorted order.

Each op is ONE persistent cooperative CUDA kernel per rank (``csrc/kernels/gmm_fused.cu``): rows move over NVLink by
peer loads / stores issued from inside the kernel that runs the tcgen05 grouped GEMM.  Without a GPU the same API
runs on a CPU engine (object all-gather + ``torch.matmul``), which is what the CPU tests exercise.

``tiling=`` names the tile shape to run; the kernel is built for one (256 x 256 x 64, see ``load_tiling_config``), so
any other request is rejected instead of being ignored.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import List, Mapping, Optional, Sequence, Tuple, Union

import torch

from ..parallel.runtime import ControlPlane, Runtime

RouteInput = Union[torch.Tensor, Sequence[int]]


# ------------------------------------------------------------------------------------------------ oracle
def reference_alltoallv_gmm(xs: Sequence[torch.Tensor], weights: Sequence[torch.Tensor], counts: Sequence[Sequence[int]],
                            num_experts: int) -> Tuple[List[torch.Tensor], List[torch.Tensor]]:
    """Plain fp32 restatement over all ranks: returns (outputs, gathered activations) per rank.

    ``counts[s][e]`` = rows rank ``s`` sends to global expert ``e``; ``xs[s]`` is sorted by expert.
    """
    world = len(xs)
    L = num_experts // world
    starts = [[sum(c[:e]) for e in range(num_experts + 1)] for c in counts]
    outs, gathered = [], []
    for d in range(world):
        rows, prods = [], []
        for l in range(L):
            e = d * L + l
            seg = [xs[s][starts[s][e]:starts[s][e + 1]] for s in range(world)]
            a = torch.cat(seg, 0) if seg else xs[0][:0]
            rows.append(a)
            prods.append((a.float() @ weights[d][l].float()).to(torch.bfloat16))
        gathered.append(torch.cat(rows, 0))
        outs.append(torch.cat(prods, 0))
    return outs, gathered


def reference_gmm_alltoallv(xs: Sequence[torch.Tensor], weights: Sequence[torch.Tensor], counts: Sequence[Sequence[int]],
                            num_experts: int) -> List[torch.Tensor]:
    """``xs[d]`` is rank ``d``'s gathered input (local expert, source rank); returns every rank's returned rows."""
    world = len(xs)
    L = num_experts // world
    n = weights[0].shape[2]
    starts = [[sum(c[:e]) for e in range(num_experts + 1)] for c in counts]
    outs = [torch.zeros((starts[s][num_experts], n), dtype=torch.bfloat16) for s in range(world)]
    for d in range(world):
        at = 0
        for l in range(L):
            e = d * L + l
            for s in range(world):
                c = counts[s][e]
                y = (xs[d][at:at + c].float() @ weights[d][l].float()).to(torch.bfloat16)
                outs[s][starts[s][e]:starts[s][e] + c] = y
                at += c
    return outs


# ------------------------------------------------------------------------------------------------ engines
class GmmEngine:
    """Launches the fused kernels for one or several (virtual) ranks that live on this GPU."""

    def __init__(self, sessions, layout, device, max_rows: int, max_k: int, max_n: int, num_experts_max: int = 1024,
                 num_sms: int = 0):
        from . import require_native

        self.C = require_native("ep_gmm_fused")
        self.sessions, self.layout, self.device = list(sessions), layout, torch.device(device)
        self.n, self.world = len(self.sessions), layout.world
        self.max_rows, self.max_k, self.max_n = int(max_rows), int(max_k), int(max_n)
        sm = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.blocks = max(1, min(num_sms or sm, sm // self.n))
        # a rank can receive every row of every rank
        self.gather_cap = self.world * self.max_rows
        self.max_tiles = self.gather_cap // 128 + num_experts_max
        i32 = dict(dtype=torch.int32, device=self.device)
        self.scratch = [dict(tile_info=torch.zeros((self.max_tiles, 4), **i32), num_tiles=torch.zeros((2,), **i32),
                             pulled=torch.zeros((self.max_tiles,), **i32), err=torch.zeros((1,), **i32),
                             gathered=None) for _ in range(self.n)]

    @staticmethod
    def region_bytes(C, max_rows: int, max_k: int, max_n: int) -> int:
        return int(C.gmm_region_bytes(max_rows, max_k, max_n))

    def symmetric_input(self, i: int, rows: int, k: int) -> torch.Tensor:
        """bf16 ``[rows, k]`` view of rank slot ``i``'s stage area: an ``x`` written here is read by the peers in place."""
        from ..models.mega_moe import _view

        if rows > self.max_rows or k > self.max_k:
            raise ValueError("the view exceeds the sizes the group was initialised with")
        off = self.layout.mega + self.C.gmm_region_offsets(self.max_rows, self.max_k, self.max_n)[2]
        return _view(self.sessions[i].workspace + off, rows * k * 2, self.device).view(torch.bfloat16).view(rows, k)

    def symmetric_output(self, i: int, rows: int, n: int) -> torch.Tensor:
        """bf16 ``[rows, n]`` view of rank slot ``i``'s receive area: ``gmm_a2av`` into it needs no final copy.  The rows
        are overwritten by the next ``gmm_a2av`` call of any rank."""
        from ..models.mega_moe import _view

        if rows > self.max_rows or n > self.max_n:
            raise ValueError("the view exceeds the sizes the group was initialised with")
        off = self.layout.mega + self.C.gmm_region_offsets(self.max_rows, self.max_k, self.max_n)[3]
        return _view(self.sessions[i].workspace + off, rows * n * 2, self.device).view(torch.bfloat16).view(rows, n)

    def _gathered(self, i: int, rows: int, k: int) -> torch.Tensor:
        buf = self.scratch[i]["gathered"]
        if buf is None or buf.numel() < rows * k:
            buf = torch.empty((max(rows, 1) * k,), dtype=torch.bfloat16, device=self.device)
            self.scratch[i]["gathered"] = buf
        return buf[:rows * k].view(rows, k)

    def _common(self, i, x, weight, counts, out, num_experts):
        sc = self.scratch[i]
        return dict(max_rows=self.max_rows, max_k=self.max_k, max_n=self.max_n, x=x.data_ptr() if x.numel() else None,
                    counts=counts.data_ptr(), out=out.data_ptr(), weight=weight.data_ptr(), rows_in=x.shape[0],
                    experts=num_experts, k=weight.shape[1], n=weight.shape[2], out_rows_cap=out.shape[0],
                    max_tiles=self.max_tiles, tile_info=sc["tile_info"].data_ptr(), num_tiles=sc["num_tiles"].data_ptr(),
                    pulled=sc["pulled"].data_ptr(), err=sc["err"].data_ptr())

    def a2av_gmm(self, xs, weights, counts, outs, gathered=None, num_experts: int = 0, stream=None) -> List[torch.Tensor]:
        """``gathered[i]`` (optional) receives the all-to-all-v result; returns the gathered buffers that were used."""
        stream = torch.cuda.current_stream(self.device) if stream is None else stream
        args, used = [], []
        for i in range(self.n):
            g = gathered[i] if gathered is not None and gathered[i] is not None else self._gathered(i, outs[i].shape[0], xs[i].shape[1])
            used.append(g)
            d = self._common(i, xs[i], weights[i], counts[i], outs[i], num_experts)
            d.update(gathered=g.data_ptr() if g.numel() else weights[i].data_ptr(), gathered_cap=g.shape[0])
            args.append(d)
        self.C.a2av_gmm(self.layout, self.sessions, args, self.blocks, stream.cuda_stream)
        return used

    def gmm_a2av(self, xs, weights, counts, outs, num_experts: int = 0, stream=None) -> None:
        stream = torch.cuda.current_stream(self.device) if stream is None else stream
        args = [self._common(i, xs[i], weights[i], counts[i], outs[i], num_experts) for i in range(self.n)]
        self.C.gmm_a2av(self.layout, self.sessions, args, self.blocks, stream.cuda_stream)

    def check(self) -> None:
        """Raises if a kernel reported a pipeline time-out (1) or row counts that do not fit (2).  Synchronises."""
        for i, sc in enumerate(self.scratch):
            code = int(sc["err"].item())
            if code:
                sc["err"].zero_()
                raise RuntimeError(f"ep_gmm_fused kernel of local rank {i} failed: " +
                                   ("a pipeline wait ran out" if code == 1 else "row counts exceed a buffer or disagree between ranks"))


@dataclass(frozen=True)
class GmmConfig:
    rank: int
    world_size: int
    max_rows: int
    max_k: int
    max_n: int
    backend: str


class _Group:
    def __init__(self, group, rank, world_size, max_rows, max_k, max_n, device, timeout, num_sms, control=None):
        self.control = control if control is not None else ControlPlane(group, rank, world_size)
        self.rank, self.world_size = self.control.rank, self.control.size
        self.max_rows, self.max_k, self.max_n = int(max_rows), int(max_k), int(max_n)
        if self.max_rows < 1 or self.max_k % 64 or self.max_n % 64 or self.max_k < 64 or self.max_n < 64:
            raise ValueError("max_rows must be positive; max_k and max_n positive multiples of 64")
        use_cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.backend = "cuda" if use_cuda else "cpu"
        self.runtime = self.engine = None
        if use_cuda:
            from . import require_native

            C = require_native("ep_gmm_fused")
            self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
            layout = C.make_mega_layout(self.world_size, 1, 128, 1, GmmEngine.region_bytes(C, self.max_rows, self.max_k, self.max_n))
            self.runtime = Runtime(self.control, layout, float(timeout), self.device)
            self.engine = GmmEngine([self.runtime.native], layout, self.device, self.max_rows, self.max_k, self.max_n, num_sms=num_sms)
        else:
            self.device = torch.device("cpu")

    def config(self) -> GmmConfig:
        return GmmConfig(self.rank, self.world_size, self.max_rows, self.max_k, self.max_n, self.backend)

    def close(self) -> None:
        if self.runtime is not None:
            self.runtime.close()
            self.runtime = None


_GROUP: Optional[_Group] = None
_PENDING: Optional[dict] = None      # a group initialised by bytes (heap_size=): sized by the first operator call
_LEASES = 0                          # udma_group contexts that are open
_CONTEXT_OWNS = False


def init_group(group=None, *, rank: Optional[int] = None, world_size: Optional[int] = None, max_rows: Optional[int] = None,
               max_k: Optional[int] = None, max_n: Optional[int] = None, device=None, timeout: float = 100.0, num_sms: int = 0,
               heap_size: Optional[int] = None, local_rank: Optional[int] = None, init_method: Optional[str] = None) -> GmmConfig:
    """Collective: allocates and exchanges the symmetric workspace (staged inputs ``[max_rows, max_k]`` and returned
    rows ``[max_rows, max_n]`` per rank).  ``max_rows`` bounds the rows a rank sends (``alltoallv_gmm``) or gets back
    (``gmm_alltoallv``) in one call.

    The reference's form (``init_udma_group(*, group, rank, world_size, local_rank, init_method, heap_size=1 << 30)``,
    ``runtime.py:87-99`` there) gives bytes instead of shapes: the workspace is then created by the first operator call,
    which knows ``k`` and ``n``: both row widths become ``max(k, n)`` rounded up to 64 and ``max_rows`` what
    ``heap_size`` bytes hold.  ``local_rank`` selects the CUDA device; ``init_method`` is accepted and unused (the ranks
    meet through ``group`` or the launcher's TCPStore)."""
    global _GROUP, _PENDING
    del init_method
    if _GROUP is not None or _PENDING is not None:
        raise RuntimeError("ep_gmm_fused group is already initialised; call destroy_group() first")
    if local_rank is not None and device is None and torch.cuda.is_available():
        device = torch.device("cuda", int(local_rank))
    shapes = (max_rows, max_k, max_n)
    if all(v is None for v in shapes):
        heap_size = (1 << 30) if heap_size is None else int(heap_size)
        if heap_size < (1 << 20):
            raise ValueError("heap_size must be at least 1 MiB")
        control = ControlPlane(group, rank, world_size)
        _PENDING = dict(control=control, group=group, rank=rank, world_size=world_size, heap_size=heap_size, device=device,
                        timeout=timeout, num_sms=num_sms)
        use_cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        return GmmConfig(control.rank, control.size, 0, 0, 0, "cuda" if use_cuda else "cpu")
    if any(v is None for v in shapes) or heap_size is not None:
        raise ValueError("pass max_rows, max_k and max_n together, or heap_size alone")
    _GROUP = _Group(group, rank, world_size, max_rows, max_k, max_n, device, timeout, num_sms)
    return _GROUP.config()


def _materialize(k: int, n: int) -> None:
    """First operator call of a group that was initialised by bytes: create the workspace for these row widths."""
    global _GROUP, _PENDING
    if _PENDING is None:
        return
    p, _PENDING = _PENDING, None
    width = -(-max(int(k), int(n)) // 64) * 64
    rows = max(1, p["heap_size"] // (4 * width))          # one staged bf16 row and one returned bf16 row per slot
    _GROUP = _Group(p["group"], p["rank"], p["world_size"], rows, width, width, p["device"], p["timeout"], p["num_sms"],
                    control=p["control"])


def check_errors() -> None:
    """Synchronise and raise if a kernel of this group reported a pipeline wait that ran out or row counts that do not fit
    (the kernels move no row in either case).  The ops call this themselves when ``DEEPEP_GMM_CHECK=1`` is set; without
    it they stay asynchronous and a caller checks at a point where a synchronisation is acceptable."""
    if _GROUP is not None and _GROUP.engine is not None:
        _GROUP.engine.check()


def _maybe_check(g) -> None:
    import os

    if g.engine is not None and os.environ.get("DEEPEP_GMM_CHECK", "0") not in ("", "0"):
        g.engine.check()


def destroy_group() -> None:
    global _GROUP, _PENDING
    if _LEASES:
        raise RuntimeError("cannot destroy the group while udma_group contexts are active")
    if _GROUP is not None:
        _GROUP.close()
        _GROUP = None
    _PENDING = None


def get_config() -> GmmConfig:
    if _GROUP is None and _PENDING is not None:
        c = _PENDING["control"]
        return GmmConfig(c.rank, c.size, 0, 0, 0, "pending")
    if _GROUP is None:
        raise RuntimeError("ep_gmm_fused group is not initialised; call init_group(...) on every rank first")
    return _GROUP.config()


init_udma_group, destroy_udma_group, get_udma_config = init_group, destroy_group, get_config
UdmaConfig = GmmConfig


@contextlib.contextmanager
def udma_group(**kwargs):
    """``with udma_group(group=ep_group): ...`` initialises the group on entry and destroys it on exit of the outermost
    context that created it; a group that was initialised explicitly is borrowed and left alone
    (parity: ``runtime.py:211-231`` of the reference)."""
    global _LEASES, _CONTEXT_OWNS
    existed = _GROUP is not None or _PENDING is not None
    config = get_config() if existed else init_group(**kwargs)
    if _LEASES == 0:
        _CONTEXT_OWNS = not existed
    _LEASES += 1
    try:
        yield config
    finally:
        _LEASES -= 1
        if _LEASES == 0 and _CONTEXT_OWNS:
            _CONTEXT_OWNS = False
            destroy_group()


def symmetric_input(rows: int, k: int) -> torch.Tensor:
    """bf16 ``[rows, k]`` view of this rank's staged-input area.  Passing it as ``x`` to :func:`alltoallv_gmm` skips
    the staging copy (the peers read it in place).  CPU engine: an ordinary tensor."""
    _materialize(k, k)
    get_config()
    if _GROUP.engine is None:
        return torch.empty((rows, k), dtype=torch.bfloat16)
    return _GROUP.engine.symmetric_input(0, rows, k)


def symmetric_output(rows: int, n: int) -> torch.Tensor:
    """bf16 ``[rows, n]`` view of this rank's returned-rows area.  Passing it as ``out`` to :func:`gmm_alltoallv` skips
    the final copy; it stays valid until the next :func:`gmm_alltoallv` call.  CPU engine: an ordinary tensor."""
    _materialize(n, n)
    get_config()
    if _GROUP.engine is None:
        return torch.empty((rows, n), dtype=torch.bfloat16)
    return _GROUP.engine.symmetric_output(0, rows, n)


TILE_SHAPE = {"m": 256, "n": 256, "k": 64}


def load_tiling_config(path=None) -> Mapping[str, int]:
    """The kernel has a single tile shape; returns it (the reference loads a measured search result here).  A JSON file
    at ``path`` is read and checked against that shape, so a configuration written for another build fails early."""
    if path is not None:
        import json

        with open(path) as fh:
            _check_tiling(json.load(fh))
    return dict(TILE_SHAPE)


def _check_tiling(tiling: Optional[Mapping[str, int]]) -> None:
    """``tiling`` may name the tile shape (keys ``m``, ``n``, ``k``; any subset): only the built shape is available."""
    if tiling is None:
        return
    if not isinstance(tiling, Mapping):
        raise TypeError("tiling must be a mapping with the keys m, n, k")
    unknown = set(tiling) - set(TILE_SHAPE)
    if unknown:
        raise ValueError(f"unknown tiling keys {sorted(unknown)}; expected a subset of {sorted(TILE_SHAPE)}")
    for key, value in tiling.items():
        if int(value) != TILE_SHAPE[key]:
            raise ValueError(f"tiling {key}={value} is not available: the kernel is built for {TILE_SHAPE}")


# ------------------------------------------------------------------------------------------------ balanced routes
def build_global_route_matrix(m: int, ep_size: int, expert_num: int) -> List[List[int]]:
    """``[source rank][global expert]`` row counts of the balanced benchmark routing: every source rank has ``m`` rows,
    every destination rank receives ``m`` rows, and inside a (source, destination) pair the rows are spread over the
    destination's local experts.  Remainders rotate: of the ``m mod ep_size`` extra rows of source ``s`` the first goes
    to rank ``s``, the next to ``s + 1``, ...; inside the pair the extra rows start at local expert ``(s + d) mod L``.
    Parity: ``build_global_route_matrix`` of the reference (``ep_gmm_fused/routing.py:24-56``), whose counts these are."""
    if m <= 0 or ep_size <= 0 or expert_num <= 0:
        raise ValueError("m, ep_size, and expert_num must be positive")
    if ep_size > 8:
        raise ValueError("ep_size must not exceed 8")
    if expert_num % ep_size:
        raise ValueError("expert_num must be divisible by ep_size")
    L = expert_num // ep_size
    if L > 64:
        raise ValueError("local expert count must not exceed 64")
    src = torch.arange(ep_size).view(-1, 1, 1)
    dst = torch.arange(ep_size).view(1, -1, 1)
    loc = torch.arange(L).view(1, 1, -1)
    pair = m // ep_size + ((dst - src) % ep_size < m % ep_size).long()              # rows of source s for destination d
    counts = pair // L + ((loc - (src + dst)) % L < pair % L).long()                # ... for local expert l of d
    matrix = counts.reshape(ep_size, expert_num)
    assert bool((matrix.sum(1) == m).all()) and bool((counts.sum((0, 2)) == m).all())
    return matrix.tolist()


def build_rank_route_tables(m: int, rank: int, ep_size: int, expert_num: int) -> Tuple[List[int], List[int]]:
    """The two flat route inputs of one rank: ``local_tokens_per_expert`` (its row of the matrix) and
    ``global_tokens_per_local_expert`` (ordered by source rank, then local expert)."""
    if not 0 <= rank < ep_size:
        raise ValueError("rank must be in [0, ep_size)")
    matrix = build_global_route_matrix(m, ep_size, expert_num)
    L = expert_num // ep_size
    return list(matrix[rank]), [matrix[s][rank * L + l] for s in range(ep_size) for l in range(L)]


def build_rank_route(m: int, rank: int, ep_size: int, expert_num: int, device):
    """``(local_tokens_per_expert, global_tokens_per_local_expert, received_rows)``: flat int64 tensors on ``device``
    plus the row count this rank receives, known on the host (pass it as ``received_rows=`` to avoid a read-back)."""
    local, received = build_rank_route_tables(m, rank, ep_size, expert_num)
    return (torch.tensor(local, dtype=torch.int64, device=device), torch.tensor(received, dtype=torch.int64, device=device),
            sum(received))


def build_rank_route_tensors(m: int, rank: int, ep_size: int, expert_num: int, device):
    local, received, _ = build_rank_route(m, rank, ep_size, expert_num, device)
    return local, received


# ------------------------------------------------------------------------------------------------ ops
def _normalize_route(route: RouteInput, name: str, expert_num: int, device) -> Tuple[torch.Tensor, Optional[List[int]]]:
    """Returns (int32 tensor on ``device``, host values or None when the route lives on a device)."""
    if isinstance(route, torch.Tensor):
        if route.dim() != 1 or route.numel() != expert_num:
            raise ValueError(f"{name} must be a flat tensor with expert_num={expert_num} elements")
        if route.dtype not in (torch.int64, torch.int32):
            raise TypeError(f"{name} must be an int64 or int32 tensor")
        host = route.tolist() if route.device.type == "cpu" else None
        return route.to(device=device, dtype=torch.int32), host
    values = [int(v) for v in route]
    if len(values) != expert_num:
        raise ValueError(f"{name} must have expert_num={expert_num} elements")
    if any(v < 0 for v in values):
        raise ValueError(f"{name} must not hold negative counts")
    return torch.tensor(values, dtype=torch.int32).to(device), values


def _check_operands(x: torch.Tensor, weight: torch.Tensor, ep_size: int, expert_num: int, cfg: GmmConfig) -> None:
    if ep_size != cfg.world_size:
        raise ValueError("TP=1 requires ep_size == group world_size")
    if expert_num <= 0 or expert_num % ep_size:
        raise ValueError("expert_num must be positive and divisible by ep_size")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("x and weight must be bf16")
    if x.dim() != 2 or weight.dim() != 3 or not x.is_contiguous() or not weight.is_contiguous():
        raise ValueError("x must be a contiguous [rows, k] tensor and weight a contiguous [local_experts, k, n] tensor")
    if weight.shape[0] != expert_num // ep_size or weight.shape[1] != x.shape[1]:
        raise ValueError("weight must have shape [expert_num / ep_size, k, n] with k == x.shape[1]")
    if x.shape[1] % 64 or weight.shape[2] % 64 or x.shape[1] > cfg.max_k or weight.shape[2] > cfg.max_n:
        raise ValueError("k and n must be multiples of 64 within the sizes the group was initialised with")


def _cpu_exchange(g: _Group, payload):
    return g.control.all_gather_object(payload)


def alltoallv_gmm(x: torch.Tensor, weight: torch.Tensor, local_tokens_per_expert: RouteInput,
                  global_tokens_per_local_expert: RouteInput, *, ep_size: int, expert_num: int,
                  received_rows: Optional[int] = None, out: Optional[torch.Tensor] = None, output_all_to_allv: bool = False,
                  all_to_allv_out: Optional[torch.Tensor] = None, tiling: Optional[Mapping[str, int]] = None):
    """Dispatch rows to their experts' ranks and apply the destination rank's grouped matmuls (one kernel)."""
    _check_tiling(tiling)
    if _PENDING is not None and x.dim() == 2 and weight.dim() == 3:
        _materialize(x.shape[1], weight.shape[2])
    g = _GROUP
    cfg = get_config()
    _check_operands(x, weight, ep_size, expert_num, cfg)
    local, local_host = _normalize_route(local_tokens_per_expert, "local_tokens_per_expert", expert_num, x.device)
    glob, glob_host = _normalize_route(global_tokens_per_local_expert, "global_tokens_per_local_expert", expert_num, x.device)
    if local_host is not None and sum(local_host) != x.shape[0]:
        raise ValueError("sum(local_tokens_per_expert) must equal x.shape[0]")
    if x.shape[0] > cfg.max_rows:
        raise ValueError(f"x has {x.shape[0]} rows; the group was initialised for at most {cfg.max_rows}")
    if received_rows is None:
        received_rows = sum(glob_host) if glob_host is not None else int(glob.sum().item())
    if received_rows < 0 or received_rows > ep_size * cfg.max_rows:
        raise ValueError("received_rows is out of range")
    if all_to_allv_out is not None and not output_all_to_allv:
        raise ValueError("all_to_allv_out requires output_all_to_allv=True")
    n, k = weight.shape[2], x.shape[1]
    if out is None:
        out = torch.empty((received_rows, n), dtype=x.dtype, device=x.device)
    elif tuple(out.shape) != (received_rows, n) or out.dtype != x.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous bf16 tensor of shape [received_rows, n]")
    if output_all_to_allv:
        if all_to_allv_out is None:
            all_to_allv_out = torch.empty((received_rows, k), dtype=x.dtype, device=x.device)
        elif tuple(all_to_allv_out.shape) != (received_rows, k) or not all_to_allv_out.is_contiguous():
            raise ValueError("all_to_allv_out must have shape [sum(global_tokens_per_local_expert), x.shape[1]]")

    if g.backend == "cpu":
        gathered = _cpu_exchange(g, (x, local.tolist()))
        outs, gath = reference_alltoallv_gmm([p[0] for p in gathered], [weight] * g.world_size, [p[1] for p in gathered], expert_num)
        # every rank multiplies by its own weights: only this rank's block of the restatement is meaningful
        if outs[g.rank].shape[0] != received_rows:
            raise ValueError("received_rows does not match the routes of the other ranks")
        out.copy_(outs[g.rank])
        if output_all_to_allv:
            all_to_allv_out.copy_(gath[g.rank])
    else:
        g.engine.a2av_gmm([x], [weight], [local], [out], [all_to_allv_out if output_all_to_allv else None], num_experts=expert_num)
        _maybe_check(g)
    return (out, all_to_allv_out) if output_all_to_allv else out


def gmm_alltoallv(x: torch.Tensor, weight: torch.Tensor, local_tokens_per_expert: RouteInput,
                  global_tokens_per_local_expert: RouteInput, *, ep_size: int, expert_num: int,
                  out: Optional[torch.Tensor] = None, tiling: Optional[Mapping[str, int]] = None) -> torch.Tensor:
    """Apply this rank's grouped matmuls and return the products to the ranks their rows came from (one kernel)."""
    _check_tiling(tiling)
    if _PENDING is not None and x.dim() == 2 and weight.dim() == 3:
        _materialize(x.shape[1], weight.shape[2])
    g = _GROUP
    cfg = get_config()
    _check_operands(x, weight, ep_size, expert_num, cfg)
    local, local_host = _normalize_route(local_tokens_per_expert, "local_tokens_per_expert", expert_num, x.device)
    glob, glob_host = _normalize_route(global_tokens_per_local_expert, "global_tokens_per_local_expert", expert_num, x.device)
    if glob_host is not None and sum(glob_host) != x.shape[0]:
        raise ValueError("sum(global_tokens_per_local_expert) must equal x.shape[0]")
    n = weight.shape[2]
    if out is None:
        rows = sum(local_host) if local_host is not None else int(local.sum().item())
        out = torch.empty((rows, n), dtype=x.dtype, device=x.device)
    elif out.dim() != 2 or out.shape[1] != n or out.dtype != x.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous bf16 tensor of shape [sum(local_tokens_per_expert), n]")
    elif local_host is not None and out.shape[0] != sum(local_host):
        raise ValueError("out must have shape [sum(local_tokens_per_expert), n]")
    if out.shape[0] > cfg.max_rows:
        raise ValueError(f"the output has {out.shape[0]} rows; the group was initialised for at most {cfg.max_rows}")

    if g.backend == "cpu":
        gathered = _cpu_exchange(g, (x, weight, local.tolist()))
        outs = reference_gmm_alltoallv([p[0] for p in gathered], [p[1] for p in gathered], [p[2] for p in gathered], expert_num)
        out.copy_(outs[g.rank])
    else:
        g.engine.gmm_a2av([x], [weight], [local], [out], num_experts=expert_num)
        _maybe_check(g)
    return out


all_to_allv_grouped_matmul = alltoallv_gmm
grouped_matmul_all_to_allv = gmm_alltoallv

__all__ = ["GmmConfig", "GmmEngine", "UdmaConfig", "udma_group", "build_global_route_matrix", "build_rank_route", "build_rank_route_tables",
           "build_rank_route_tensors", "all_to_allv_grouped_matmul", "alltoallv_gmm", "check_errors", "destroy_group", "destroy_udma_group",
           "get_config", "get_udma_config", "gmm_alltoallv", "grouped_matmul_all_to_allv", "init_group", "init_udma_group",
           "load_tiling_config", "reference_alltoallv_gmm", "reference_gmm_alltoallv", "symmetric_input", "symmetric_output"]
