"""``ElasticBuffer`` and ``EPHandle``: the public expert-parallel dispatch/combine API.

Parity with the reference (``deep_ep/backends/mesh_clos/elastic.py``):
``EPHandle`` :88-173, constructor :178-269, ``get_buffer_size_hint`` :279-314,
``barrier`` :316-326, ``capture``/``get_comm_stream`` :329-341, low-latency
selection :401-451 and :709-747, ``dispatch`` :648-1008, ``combine``
:1010-1283, call-signature preflight :45-72; and with the Direct backend's
wider option set (``deep_ep/backends/direct/elastic.py:641-1162``:
``do_expand=False``, ``expert_alignment``, ``do_cpu_sync=False``, statistics,
``bias``), which this implementation also accepts.

One buffer serves one process group of 1, 2, 4 or 8 GPUs on one NVLink
domain.  Work is issued on the buffer's private communication stream; see
``_enter``/``_leave`` for the ordering rules.
"""
from __future__ import annotations

from typing import Any, List, Optional, Sequence, Tuple

import torch

from .._compat import (CALL_ALIASES, COMBINE_ALIASES, ELASTIC_INIT_ALIASES, ESTIMATOR_ALIASES, HANDLE_ALIASES, QPS_ALIASES,
                       keyword_aliases)
from ..utils.event import EventHandle, EventOverlap
from . import layout as L
from .runtime import ControlPlane, Runtime
from .streams import get_global_comm_stream

METADATA_VERSION = 1
_next_buffer_id = 0


def _unavailable(name: str):
    raise NotImplementedError(f"{name} is outside the scope of this expert-parallel library")


class EPHandle:
    """Routing plan of one dispatch; owned by one buffer, reusable until the matching backward is done."""

    def __init__(self, do_expand, num_experts, expert_alignment, num_max_tokens_per_rank, num_sms, topk_idx,
                 num_recv_tokens, num_expanded_tokens, num_recv_tokens_per_expert_list,
                 psum_num_recv_tokens_per_scaleup_rank, psum_num_recv_tokens_per_expert,
                 num_unaligned_recv_tokens_per_expert, recv_src_metadata, dst_buffer_slot_idx, token_metadata_at_forward,
                 channel_linked_list, is_low_latency=False):
        self.do_expand = do_expand
        self.num_experts = num_experts
        self.expert_alignment = expert_alignment
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.num_sms = num_sms
        self.topk_idx = topk_idx
        self.num_recv_tokens = num_recv_tokens
        self.num_expanded_tokens = num_expanded_tokens
        self.num_recv_tokens_per_expert_list = num_recv_tokens_per_expert_list
        self.psum_num_recv_tokens_per_scaleup_rank = psum_num_recv_tokens_per_scaleup_rank
        self.psum_num_recv_tokens_per_expert = psum_num_recv_tokens_per_expert
        self.num_unaligned_recv_tokens_per_expert = num_unaligned_recv_tokens_per_expert
        self.recv_src_metadata = recv_src_metadata
        self.dst_buffer_slot_idx = dst_buffer_slot_idx
        self.token_metadata_at_forward = token_metadata_at_forward
        self.channel_linked_list = channel_linked_list
        self.is_low_latency = is_low_latency
        # private: set by the buffer that created the handle
        self.metadata_version = METADATA_VERSION
        self.dedup_group_size = 1          # rank-level dedup: a token crosses the link once per destination GPU
        self._plan = None
        self._buffer_id = None
        self._tokens = 0
        self._hidden = 0
        self._owner = None                 # the buffer that made the handle
        self._saved_weights = None         # low-latency: source weights applied by combine
        self._snapshots: Tuple = ()

    @staticmethod
    def _stamp(t: torch.Tensor):
        # inference tensors (created under torch.inference_mode) keep no version counter: only their storage is compared
        return t.data_ptr(), (None if t.is_inference() else t._version)

    def _snapshot(self) -> None:
        self._snapshots = tuple(self._stamp(t) for t in self._tracked())

    def _tracked(self) -> List[torch.Tensor]:
        return [] if self._plan is None else list(self._plan.tensors())

    def _check_unchanged(self) -> None:
        now = tuple(self._stamp(t) for t in self._tracked())
        if now != self._snapshots:
            raise RuntimeError("handle metadata (or its topk_idx) was modified in place after dispatch")


def _timeout_seconds(default: float) -> float:
    """Device wait limit: ``DEEPEP_GPU_TIMEOUT_SECONDS`` (alias ``DEEPEP_NPU_TIMEOUT_SECONDS``) overrides the constructor."""
    import os

    for name in ("DEEPEP_GPU_TIMEOUT_SECONDS", "DEEPEP_NPU_TIMEOUT_SECONDS"):
        if name in os.environ:
            value = float(os.environ[name])
            if not 1 <= value <= 3600:
                raise ValueError(f"{name} must be in [1, 3600] seconds")
            return value
    return default


def _as_event(ev) -> Optional[EventHandle]:
    if ev is None:
        return None
    if isinstance(ev, EventOverlap):
        return ev.event
    return ev


class ElasticBuffer:
    """Symmetric workspace plus dispatch/combine over it."""

    def __init__(self, group=None, num_bytes=None, num_cpu_bytes=0, num_max_tokens_per_rank=0, hidden=0, num_topk=0,
                 use_fp8_dispatch=False, deterministic=False, allow_hybrid_mode=True, allow_multiple_reduction=True,
                 prefer_overlap_with_compute=True, sl_idx=3, num_allocated_qps=0, num_cpu_timeout_secs=300,
                 num_gpu_timeout_secs=100, explicitly_destroy=False, *, rank=None, world_size=None, bootstrap="default",
                 combine_only=False, use_1g_huge_pages=True, debug_collectives=False, machine_type="auto",
                 rootinfo_path=None, device=None, num_sms=0, comm_stream=None):
        global _next_buffer_id
        del num_cpu_bytes, allow_hybrid_mode, allow_multiple_reduction, prefer_overlap_with_compute, sl_idx
        del num_allocated_qps, use_1g_huge_pages, rootinfo_path, combine_only
        if machine_type not in ("auto", None, "nvswitch", "b200", "single", "cpu"):
            raise ValueError("machine_type must be 'auto', 'nvswitch', 'single' or 'cpu': one NVLink/NVSwitch domain is the "
                             "only multi-GPU topology")
        if bootstrap not in ("default", "auto", "group", "store"):
            raise ValueError("bootstrap must be 'default', 'group' or 'store'")
        if isinstance(comm_stream, str) and comm_stream != "global":
            raise ValueError("comm_stream must be None (a stream of this buffer's own), 'global' (the stream that "
                             "get_global_comm_stream returns, shared by every buffer of the process) or a CUDA stream")
        if num_max_tokens_per_rank <= 0 or hidden <= 0 or num_topk <= 0:
            raise ValueError("num_max_tokens_per_rank, hidden and num_topk are required")
        for name, value in (("num_gpu_timeout_secs", num_gpu_timeout_secs), ("num_cpu_timeout_secs", num_cpu_timeout_secs)):
            if not 1 <= float(value) <= 3600:
                raise ValueError(f"{name} must be in [1, 3600] seconds")
        if num_max_tokens_per_rank > L.MAX_TOKENS or num_topk > L.MAX_TOPK:
            raise ValueError(f"limits: tokens <= {L.MAX_TOKENS}, top-k <= {L.MAX_TOPK}")
        L.validate_hidden(hidden, use_fp8_dispatch)
        self.control = ControlPlane(group, rank, world_size, bootstrap, timeout=float(num_cpu_timeout_secs))
        self.group, self.rank, self.world_size = group, self.control.rank, self.control.size
        if self.world_size not in L.WORLD_SIZES:
            raise ValueError(f"world size must be one of {L.WORLD_SIZES}")
        self.num_max_tokens_per_rank, self.hidden, self.num_topk = num_max_tokens_per_rank, hidden, num_topk
        self.use_fp8_dispatch, self.deterministic = bool(use_fp8_dispatch), bool(deterministic)
        self.explicitly_destroy, self.debug_collectives = bool(explicitly_destroy), bool(debug_collectives)
        self.num_cpu_timeout_secs, self.num_gpu_timeout_secs = num_cpu_timeout_secs, num_gpu_timeout_secs
        self.num_sms = num_sms
        self._id, _next_buffer_id = _next_buffer_id, _next_buffer_id + 1
        self._destroyed = False
        needed = L.elastic_size_hint(self.world_size, num_max_tokens_per_rank, hidden, num_topk)
        # Capacity fallback (parity: deep_ep/buffers/_combine_reuse.py of the reference): a workspace capped below the size
        # hint keeps the partials of a window of tokens only, and combine runs one pass per window.
        self.combine_window = 0
        if num_bytes not in (None, 0) and num_bytes < needed:
            try:
                self.combine_window = L.combine_window(self.world_size, num_max_tokens_per_rank, hidden, num_topk, int(num_bytes))
            except ValueError as exc:
                raise ValueError(f"num_bytes={num_bytes} is too small for this shape ({exc}); get_buffer_size_hint gives "
                                 f"{needed}") from None
            needed = L.workspace_bytes(self.world_size, num_max_tokens_per_rank, hidden, num_topk,
                                       L.ll_region_bytes(self.world_size, num_max_tokens_per_rank, hidden, num_topk),
                                       0, self.combine_window)
        self.num_bytes = needed if num_bytes in (None, 0) or self.combine_window else int(num_bytes)
        self.on_cuda = torch.cuda.is_available() and (
            self.control.backend() != "gloo" or (device is not None and torch.device(device).type == "cuda"))
        self.runtime: Optional[Runtime] = None
        # what the ranks run on: detected on every rank, exchanged and checked by all of them before memory is shared
        from . import topology

        cuda_device = None
        if self.on_cuda:
            cuda_device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.machine_type, self.machine_selection = topology.agree(self.control, cuda_device, machine_type, details=True)
        if self.on_cuda:
            from ..ops import require_native
            from .engine_cuda import CudaEngine

            C = require_native("ElasticBuffer")
            self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
            ll = L.ll_region_bytes(self.world_size, num_max_tokens_per_rank, hidden, num_topk)
            self.layout = C.make_layout(self.world_size, num_max_tokens_per_rank, hidden, num_topk, ll, 0, self.combine_window)
            assert self.layout.total == needed, "native and Python workspace layouts disagree"
            self.runtime = Runtime(self.control, self.layout, float(_timeout_seconds(num_gpu_timeout_secs)), self.device,
                                   comm_stream=comm_stream)
            from ..utils.hostwait import cpu_timeout_seconds

            self.engine = CudaEngine([self.runtime.native], self.layout, self.device, num_sms=num_sms,
                                     host_timeout=cpu_timeout_seconds(num_cpu_timeout_secs))
        else:
            from .engine_cpu import CpuEngine

            self.device = torch.device("cpu")
            self.layout = None
            self.engine = CpuEngine(self.control, num_max_tokens_per_rank, hidden, num_topk)
        self._failed = False

    # ------------------------------------------------------------------ sizing and topology
    @staticmethod
    def get_buffer_size_hint(group, num_max_tokens_per_rank, hidden, num_topk=0, use_fp8_dispatch=False,
                             allow_hybrid_mode=True, allow_multiple_reduction=True, *, world_size=None,
                             machine_type="auto", rootinfo_path=None) -> int:
        """Bytes of symmetric workspace for this shape (2 MiB aligned)."""
        del use_fp8_dispatch, allow_hybrid_mode, allow_multiple_reduction, machine_type, rootinfo_path
        if world_size is None:
            world_size = ControlPlane(group).size
        return L.elastic_size_hint(world_size, num_max_tokens_per_rank, hidden, max(1, num_topk))

    def get_physical_domain_size(self) -> Tuple[int, int]:
        return 1, self.world_size

    def get_logical_domain_size(self) -> Tuple[int, int]:
        return 1, self.world_size

    # ------------------------------------------------------------------ device phase timing
    def enable_profiling(self, on: bool = True) -> None:
        """Time every kernel this buffer launches with CUDA events (also switched on by ``DEEPEP_PROFILE=1``)."""
        if hasattr(self.engine, "enable_profiling"):
            self.engine.enable_profiling(on)

    def pop_profile(self):
        """``[(kernel, microseconds)]`` recorded since the last call; empty on engines without device timing."""
        return self.engine.pop_timings() if hasattr(self.engine, "pop_timings") else []

    def get_theoretical_num_sms(self, num_experts, num_topk, num_scaleout_topk=0, rdma_gbs=0, nvlink_gbs=0,
                                sm_read_gbs=200, sm_write_gbs=50) -> int:
        """SMs needed to keep NVLink busy, from per-SM copy rates (bulk-copy engines move the rows)."""
        del num_experts, num_scaleout_topk, rdma_gbs
        from ..utils.envs import get_nvlink_gbs

        link = nvlink_gbs or get_nvlink_gbs()
        per_token_copies = min(num_topk, self.world_size)
        send = -(-link // max(1, sm_write_gbs * 2))
        recv = -(-link * max(1, num_topk) // (per_token_copies * max(1, sm_read_gbs)))
        return int(min(128, max(8, send + recv)))

    get_theoretical_num_compute_units = get_theoretical_num_sms

    def get_theoretical_num_qps(self, num_sms) -> int:
        del num_sms
        return 0  # loads/stores through mapped peer memory need no queue pairs

    # features of upstream DeepEP that are explicitly outside this library
    def engram_write(self, *a, **k): _unavailable("Engram")
    def engram_fetch(self, *a, **k): _unavailable("Engram")
    def pp_set_config(self, *a, **k): _unavailable("pipeline parallelism")
    def pp_send(self, *a, **k): _unavailable("pipeline parallelism")
    def pp_recv(self, *a, **k): _unavailable("pipeline parallelism")
    def all_gather(self, *a, **k): _unavailable("AGRS all_gather")
    def reduce_scatter(self, *a, **k): _unavailable("AGRS reduce_scatter")

    # ------------------------------------------------------------------ lifecycle
    def destroy(self) -> None:
        """Collective: waits for all ranks, then frees the workspace.  Idempotent."""
        if self._destroyed:
            return
        self._destroyed = True
        if self.runtime is not None:
            self.runtime.close()
        else:
            self.control.barrier()

    def _alive(self) -> None:
        if self._destroyed:
            raise RuntimeError("the buffer was destroyed")
        if self._failed:
            raise RuntimeError("A previous communication launch failed; restart the distributed job")
        if self.runtime is not None:
            self.runtime.ensure_alive()

    def get_comm_stream(self):
        self._alive()
        return self.runtime.stream if self.runtime is not None else None

    @staticmethod
    def capture() -> EventHandle:
        return EventHandle()

    def barrier(self, use_comm_stream: bool = True, with_cpu_sync: bool = False, sequential: bool = True) -> None:
        del sequential
        self._alive()
        if self.runtime is None:
            self.control.barrier()
            return
        stream = self.runtime.stream if use_comm_stream else torch.cuda.current_stream(self.device)
        if use_comm_stream:
            stream.wait_stream(torch.cuda.current_stream(self.device))
        self.engine.barrier(stream=stream)
        if use_comm_stream:
            torch.cuda.current_stream(self.device).wait_stream(stream)
        if with_cpu_sync:
            stream.synchronize()
            self._check()

    # ------------------------------------------------------------------ stream / event ordering
    def _enter(self, previous_event, previous_event_before_epilogue):
        """The comm stream starts after ``previous_event`` (or after everything queued on the current stream)."""
        if self.runtime is None:
            return None
        comm, cur = self.runtime.stream, torch.cuda.current_stream(self.device)
        waited = False
        for ev in (previous_event, previous_event_before_epilogue):
            h = _as_event(ev)
            if h is not None:
                comm.wait_event(h.event)
                waited = True
        if not waited:
            comm.wait_stream(cur)
        return comm

    @staticmethod
    def _allocates_on_comm(allocate_on_comm_stream: bool, *events) -> bool:
        """Outputs come from the communication stream's memory pool when the caller asks for it, and also whenever the
        call is ordered after an event instead of after the current stream: a block that the current stream's pool
        hands out may still be read by kernels queued there after that event was recorded, and the communication
        kernels, which only wait for the event, would overwrite it under them."""
        return bool(allocate_on_comm_stream) or any(_as_event(e) is not None for e in events)

    def _leave(self, comm, async_with_compute_stream: bool, resources: Sequence[Any],
               allocated_on_comm: bool = False) -> EventOverlap:
        """Sync mode: the current stream waits for the call.  Async mode: the caller waits on the returned event."""
        if comm is None:
            return EventOverlap()
        cur = torch.cuda.current_stream(self.device)
        if async_with_compute_stream:
            return EventOverlap._from_resources(EventHandle(comm), tuple(resources))
        cur.wait_stream(comm)
        if allocated_on_comm:
            # The outputs belong to the communication stream's memory pool but will be used on the current stream: tell
            # the allocator, or it could hand a dropped block to the next communication kernel while compute still reads it.
            for t in resources:
                if isinstance(t, torch.Tensor) and t.is_cuda:
                    t.record_stream(cur)
        # otherwise outputs were allocated on the current stream, which now waits for the call: stream-ordered reuse of
        # their memory is already safe
        return EventOverlap()

    def _check(self) -> None:
        try:
            self.engine.check_status()
        except Exception:
            self._failed = True
            if self.runtime is not None:
                self.runtime.failed = True
            raise

    def _preflight(self, phase: str, signature: Sequence[int]) -> None:
        """debug_collectives: every rank must be making the same call with compatible arguments."""
        if not self.debug_collectives:
            return
        rows = self.control.all_gather_object((phase, tuple(int(v) for v in signature)))
        if any(r != rows[0] for r in rows):
            raise RuntimeError(f"ranks disagree on the {phase} call: {rows}")

    # ------------------------------------------------------------------ dispatch
    def _wants_low_latency(self, handle, topk_weights, tokens, num_max, expert_alignment, stats, num_sms,
                           do_zero_padding, col_major_sf, do_expand) -> bool:
        """Low latency serves a fresh dispatch with weights and default options on a buffer of at most 256 tokens.

        ``do_expand=True`` always selects the high-throughput path (whose combine does not apply weights).
        """
        if handle is not None or topk_weights is None or stats is not None or num_sms or do_expand:
            return False
        if expert_alignment not in (None, 1) or do_zero_padding or col_major_sf:
            return False
        m = num_max or self.num_max_tokens_per_rank
        # nothing here may depend on this rank's own batch (an empty batch included): all ranks must choose alike
        return tokens <= m <= L.LL_MAX_TOKENS and self.num_max_tokens_per_rank <= L.LL_MAX_TOKENS

    def dispatch(self, x, topk_idx=None, topk_weights=None, cumulative_local_expert_recv_stats=None, num_experts=None,
                 num_max_tokens_per_rank=None, expert_alignment=None, num_sms=0, num_qps=0, previous_event=None,
                 previous_event_before_epilogue=None, async_with_compute_stream=False, allocate_on_comm_stream=False,
                 handle=None, do_handle_copy=True, do_cpu_sync=None, do_expand=False, do_zero_padding=False,
                 use_tma_aligned_col_major_sf=False, _rank_matrix=False):
        """Send every token to the ranks that own its experts.

        Returns ``(recv_x | (recv_x, recv_x_sf), recv_topk_idx, recv_topk_weights, handle, event)``.
        """
        del num_qps
        self._alive()
        x_data, x_sf = (x if isinstance(x, (tuple, list)) else (x, None))
        # Scales travel bit for bit, so int32 scales (four ue8m0 exponents per 128 values, the MXFP8 form) are carried as
        # the fp32 words they occupy and handed back as int32.
        packed = x_sf is not None and x_sf.dtype == torch.int32
        if packed:
            x_sf = x_sf.view(torch.float32)
            x = (x_data, x_sf)
        self._validate_x(x_data, x_sf)
        tokens = x_data.shape[0]
        if handle is not None:
            if topk_idx is not None or topk_weights is not None:
                raise ValueError("pass either routing tensors or a handle, not both")
            return self._dispatch_cached(x_data, x_sf, handle, num_sms, previous_event, previous_event_before_epilogue,
                                         async_with_compute_stream, allocate_on_comm_stream, packed)
        if topk_idx is None or num_experts is None:
            raise ValueError("a fresh dispatch needs topk_idx and num_experts")
        self._validate_routing(topk_idx, topk_weights, tokens, num_experts)
        stats = cumulative_local_expert_recv_stats
        low_latency = self._wants_low_latency(handle, topk_weights, tokens, num_max_tokens_per_rank, expert_alignment, stats,
                                              num_sms, do_zero_padding, use_tma_aligned_col_major_sf, do_expand)
        low_latency = low_latency and hasattr(self.engine, "ll_combine")
        # do_expand=None is the reference's "not given": its fresh dispatch is expanded then (upstream's default, False,
        # gives the rank layout)
        expand = True if (low_latency or do_expand is None) else bool(do_expand)
        alignment = 1 if expert_alignment is None else int(expert_alignment)
        if alignment < 1:
            raise ValueError("expert_alignment must be positive")
        if alignment > 1 and not expand:
            raise ValueError("expert_alignment needs do_expand=True")
        cpu_sync = True if do_cpu_sync is None else bool(do_cpu_sync)
        mode = self._mode(x_data, x_sf)
        self._preflight("dispatch", (tokens > self.num_max_tokens_per_rank, self.hidden, self.num_topk, num_experts, expand,
                                     alignment, mode, low_latency, cpu_sync))
        comm = self._enter(previous_event, previous_event_before_epilogue)
        allocate_on_comm_stream = self._allocates_on_comm(allocate_on_comm_stream, previous_event, previous_event_before_epilogue)
        if do_handle_copy and topk_idx.is_inference():
            # The handle watches ordinary tensors for in-place changes through their version counters.  An inference tensor
            # (torch.inference_mode) has none, so the handle keeps a copy of its own instead; do_handle_copy=False leaves
            # it to the caller to keep the indices unchanged while the handle lives.
            with self._on(comm):
                topk_idx = topk_idx.clone()
        try:
            with self._on(comm if allocate_on_comm_stream else None):
                if low_latency and hasattr(self.engine, "ll_dispatch"):
                    return self._dispatch_low_latency(x_data, x_sf, topk_idx, topk_weights, num_experts, mode, cpu_sync,
                                                      comm, async_with_compute_stream, allocate_on_comm_stream, packed)
                plan = self.engine.notify([topk_idx], [topk_weights], num_experts, expand=expand, alignment=alignment,
                                          cpu_sync=cpu_sync, stream=comm, **({"rank_matrix": True} if _rank_matrix else {}))[0]
                recv_x, recv_sf = self.engine.dispatch([x if x_sf is not None else x_data], [plan], mode,
                                                       blocks=num_sms or self.num_sms, stream=comm)[0]
                if stats is not None:
                    with self._on(comm):   # the counts are produced on the communication stream
                        stats.add_(plan.expert_counts.to(stats.dtype).to(stats.device))
        except Exception as exc:
            self._note_failure(exc)
            raise
        rows = plan.num_rows
        recv_w = plan.recv_w[:rows] if plan.recv_w is not None else None
        recv_idx = None if expand else plan.recv_idx[:rows]
        h = self._make_handle(plan, expand, num_experts, alignment, num_sms, topk_idx, tokens, low_latency)
        if low_latency:
            h._saved_weights = topk_weights
        if recv_sf is not None and use_tma_aligned_col_major_sf:
            recv_sf = _col_major(recv_sf)
        out_x = recv_x if recv_sf is None else (recv_x, recv_sf.view(torch.int32) if packed else recv_sf)
        event = self._leave(comm, async_with_compute_stream, [recv_x, recv_sf, recv_w, recv_idx, x_data, x_sf, topk_idx,
                                                               topk_weights] + h._tracked(), allocate_on_comm_stream)
        return out_x, recv_idx, recv_w, h, event

    def _note_failure(self, exc: Exception) -> None:
        """A failed launch or a wait that ran out leaves ranks out of step: poison the buffer."""
        if type(exc).__name__ == "CommunicationError":
            self._failed = True
            if self.runtime is not None:
                self.runtime.failed = True

    def _dispatch_cached(self, x_data, x_sf, handle: EPHandle, num_sms, previous_event, previous_event_before_epilogue,
                         async_with_compute_stream, allocate_on_comm_stream=False, packed=False):
        self._own(handle)
        handle._check_unchanged()
        if x_data.shape[0] != handle._tokens:
            raise ValueError("a cached dispatch must carry the token count of the original dispatch")
        mode = self._mode(x_data, x_sf)
        self._preflight("cached_dispatch", (x_data.shape[0] > 0, self.hidden, mode))
        comm = self._enter(previous_event, previous_event_before_epilogue)
        allocate_on_comm_stream = self._allocates_on_comm(allocate_on_comm_stream, previous_event, previous_event_before_epilogue)
        with self._on(comm if allocate_on_comm_stream else None):
            if handle.is_low_latency and hasattr(self.engine, "ll_dispatch"):
                recv_x, recv_sf = self.engine.ll_dispatch_cached([x_data if x_sf is None else (x_data, x_sf)], [handle._plan],
                                                                 mode, stream=comm)[0]
            else:
                recv_x, recv_sf = self.engine.dispatch([x_data if x_sf is None else (x_data, x_sf)], [handle._plan], mode,
                                                       blocks=num_sms or self.num_sms, stream=comm)[0]
        out_x = recv_x if recv_sf is None else (recv_x, recv_sf.view(torch.int32) if packed else recv_sf)
        event = self._leave(comm, async_with_compute_stream, [recv_x, recv_sf, x_data, x_sf] + handle._tracked(),
                            allocate_on_comm_stream)
        return out_x, None, None, handle, event

    def _dispatch_low_latency(self, x_data, x_sf, topk_idx, topk_weights, num_experts, mode, cpu_sync, comm,
                              async_with_compute_stream, allocated_on_comm=False, packed=False):
        plan, recv_x, recv_sf = self.engine.ll_dispatch([x_data if x_sf is None else (x_data, x_sf)], [topk_idx],
                                                        [topk_weights], num_experts, mode, cpu_sync=cpu_sync, stream=comm)[0]
        rows = plan.num_rows
        h = self._make_handle(plan, True, num_experts, 1, 0, topk_idx, x_data.shape[0], True)
        h._saved_weights = topk_weights
        recv_w = plan.recv_w[:rows]
        out_x = recv_x if recv_sf is None else (recv_x, recv_sf.view(torch.int32) if packed else recv_sf)
        event = self._leave(comm, async_with_compute_stream, [recv_x, recv_sf, recv_w, x_data, x_sf, topk_idx, topk_weights]
                            + h._tracked(), allocated_on_comm)
        return out_x, None, recv_w, h, event

    def _make_handle(self, plan, expand, num_experts, alignment, num_sms, topk_idx, tokens, low_latency) -> EPHandle:
        counts = plan.expert_counts_list
        h = EPHandle(expand, num_experts, alignment, self.num_max_tokens_per_rank, num_sms, topk_idx,
                     plan.num_staged_rows, plan.num_rows, counts,
                     None if plan.rank_rows is None else plan.rank_rows[1:], plan.expert_offsets[1:],
                     plan.expert_counts, plan.recv_row_src, getattr(plan, "slot_row", None),
                     getattr(plan, "stage_meta", None), getattr(plan, "chunk_start", None), is_low_latency=low_latency)
        h._plan, h._buffer_id, h._tokens, h._hidden = plan, self._id, tokens, self.hidden
        h._owner = self      # a live handle keeps its buffer alive (replacing the caller's variable does not end the buffer)
        h._snapshot()
        return h

    # ------------------------------------------------------------------ combine
    def combine(self, x, handle, topk_weights=None, bias=None, num_sms=0, num_qps=0, previous_event=None,
                previous_event_before_epilogue=None, async_with_compute_stream=False, allocate_on_comm_stream=False,
                combine_num_sms: int = 0, reduce_num_sms: int = 0):
        """Return every expert output row to its source token and reduce.

        ``combine_num_sms`` / ``reduce_num_sms`` (both or neither) set how many SMs return rows on the expert side and
        how many reduce at the source; by default ``num_sms`` is divided 72 / 28.

        High-throughput handles: unweighted fp32 sum (bf16 partial per expert rank), optional ``bias`` (a tensor or a
        pair) added at the source, optional fp32 ``topk_weights`` returned per slot as an independent channel.
        Low-latency handles: ``sum_k w_k * row_k`` with the weights saved at dispatch.
        Returns ``(combined_x, combined_topk_weights | None, event)``.
        """
        del num_qps
        self._alive()
        self._own(handle)
        handle._check_unchanged()
        plan = handle._plan
        if not isinstance(x, torch.Tensor) or x.dim() != 2 or x.shape[1] != self.hidden or x.dtype != torch.bfloat16:
            raise ValueError(f"combine expects a bf16 [rows, {self.hidden}] tensor")
        if x.shape[0] != plan.num_rows:
            raise ValueError(f"combine expects {plan.num_rows} rows (the dispatch output), got {x.shape[0]}")
        if not x.is_contiguous():
            raise ValueError("combine input must be contiguous")
        if topk_weights is not None:
            want = (plan.num_rows,) if plan.expand else (plan.num_rows, self.num_topk)
            if tuple(topk_weights.shape) != want or topk_weights.dtype != torch.float32:
                raise ValueError(f"topk_weights must be fp32 of shape {want}")
        biases = bias if isinstance(bias, (tuple, list)) else (bias, None)
        for b in biases:
            if b is not None and (tuple(b.shape) != (handle._tokens, self.hidden) or b.dtype != torch.bfloat16):
                raise ValueError("bias must be bf16 [tokens, hidden]")
        self._preflight("combine", (self.hidden, plan.expand, topk_weights is not None, bias is not None,
                                    handle.is_low_latency))
        for name, v in (("combine_num_sms", combine_num_sms), ("reduce_num_sms", reduce_num_sms)):
            if not isinstance(v, int) or isinstance(v, bool) or v < 0:
                raise ValueError(f"{name} must be a nonnegative integer")
        if bool(combine_num_sms) != bool(reduce_num_sms):
            raise ValueError("pass combine_num_sms and reduce_num_sms together")
        split = (combine_num_sms, reduce_num_sms) if combine_num_sms else None
        if split is not None and (handle.is_low_latency or not hasattr(self.engine, "split_blocks")):
            split = None                      # one kernel role per SM only exists on the high-throughput CUDA path
        comm = self._enter(previous_event, previous_event_before_epilogue)
        allocate_on_comm_stream = self._allocates_on_comm(allocate_on_comm_stream, previous_event, previous_event_before_epilogue)
        with self._on(comm if allocate_on_comm_stream else None):
            if handle.is_low_latency:
                if topk_weights is not None or bias is not None:
                    raise ValueError("a low-latency combine applies the weights saved at dispatch; pass neither weights nor bias")
                out, out_w = self.engine.ll_combine([x], [plan], stream=comm)[0], None
            else:
                out, out_w = self.engine.combine([x], [plan], [topk_weights], bias=None if bias is None else [tuple(biases)],
                                                 blocks=num_sms or self.num_sms, stream=comm,
                                                 **({"split": split} if split is not None else {}))[0]
        event = self._leave(comm, async_with_compute_stream, [out, out_w, x, topk_weights] + [b for b in biases if b is not None]
                            + handle._tracked(), allocate_on_comm_stream)
        return out, out_w, event

    # ------------------------------------------------------------------ validation helpers
    def _on(self, comm):
        import contextlib

        return torch.cuda.stream(comm) if comm is not None else contextlib.nullcontext()

    def _own(self, handle) -> None:
        if not isinstance(handle, EPHandle) or handle._plan is None:
            raise TypeError("handle must be an EPHandle returned by dispatch")
        if handle._buffer_id != self._id:
            raise ValueError("the handle belongs to another buffer")

    def _mode(self, x_data, x_sf) -> int:
        if x_sf is not None:
            return 1
        return 2 if self.use_fp8_dispatch else 0

    def _validate_x(self, x_data, x_sf) -> None:
        if not isinstance(x_data, torch.Tensor) or x_data.dim() != 2 or x_data.shape[1] != self.hidden:
            raise ValueError(f"x must be a [tokens, {self.hidden}] tensor")
        if not x_data.is_contiguous():
            raise ValueError("x must be contiguous")
        if x_data.shape[0] > self.num_max_tokens_per_rank:
            raise ValueError(f"{x_data.shape[0]} tokens exceed num_max_tokens_per_rank={self.num_max_tokens_per_rank}")
        if self.on_cuda != x_data.is_cuda:
            raise ValueError("x lives on the wrong device for this buffer")
        if x_sf is None:
            if x_data.dtype not in (torch.bfloat16, torch.float16):
                raise ValueError("x must be bf16/fp16, or an (e4m3, fp32 scales) pair")
            if self.use_fp8_dispatch and x_data.dtype != torch.bfloat16:
                raise ValueError("the fused fp8 dispatch quantises bf16 input")
        else:
            if x_data.dtype != torch.float8_e4m3fn or x_sf.dtype != torch.float32:
                raise ValueError("the fp8 pair must be (float8_e4m3fn [T, H], float32 or int32 [T, H / 128])")
            if self.hidden % 128 or tuple(x_sf.shape) != (x_data.shape[0], self.hidden // 128) or not x_sf.is_contiguous():
                raise ValueError("scales must be contiguous [tokens, hidden / 128]")

    def _validate_routing(self, topk_idx, topk_weights, tokens, num_experts) -> None:
        if topk_idx.dtype != torch.int64 or tuple(topk_idx.shape) != (tokens, self.num_topk) or not topk_idx.is_contiguous():
            raise ValueError(f"topk_idx must be contiguous int64 [{tokens}, {self.num_topk}]")
        if topk_weights is not None and (topk_weights.dtype != torch.float32 or tuple(topk_weights.shape) != (tokens, self.num_topk)
                                         or not topk_weights.is_contiguous()):
            raise ValueError(f"topk_weights must be contiguous fp32 [{tokens}, {self.num_topk}]")
        if num_experts <= 0 or num_experts % self.world_size or num_experts > 1024:
            raise ValueError("num_experts must be a positive multiple of the world size, at most 1024")


def _col_major(sf: torch.Tensor) -> torch.Tensor:
    """[R, C] scales stored column-major with the row count padded to 4 (16-byte columns)."""
    rows, cols = sf.shape
    padded = -(-rows // 4) * 4
    store = torch.zeros((cols, padded), dtype=sf.dtype, device=sf.device)
    store[:, :rows] = sf.t()
    return store.t()[:rows]


ElasticBuffer.__init__ = keyword_aliases(ElasticBuffer.__init__, ELASTIC_INIT_ALIASES)
ElasticBuffer.dispatch = keyword_aliases(ElasticBuffer.dispatch, CALL_ALIASES)
ElasticBuffer.combine = keyword_aliases(ElasticBuffer.combine, COMBINE_ALIASES)
ElasticBuffer.get_theoretical_num_sms = keyword_aliases(ElasticBuffer.get_theoretical_num_sms, ESTIMATOR_ALIASES)
ElasticBuffer.get_theoretical_num_compute_units = ElasticBuffer.get_theoretical_num_sms
ElasticBuffer.get_theoretical_num_qps = keyword_aliases(ElasticBuffer.get_theoretical_num_qps, QPS_ALIASES)
EPHandle.__init__ = keyword_aliases(EPHandle.__init__, HANDLE_ALIASES)
# the platform-neutral spelling of the handle's SM budget reads and writes the same value
EPHandle.num_compute_units = property(lambda self: self.num_sms, lambda self, value: setattr(self, "num_sms", value))

__all__ = ["ElasticBuffer", "EPHandle", "get_global_comm_stream"]
