"""``Buffer``: upstream DeepEP's V1 interface (``get_dispatch_layout`` / ``dispatch`` / ``combine``).

Parity: ``deep_ep/backends/direct/buffer.py`` of the reference (``get_dispatch_layout`` :420-463,
``dispatch`` :465-680 with the six-tensor handle, ``num_worst_tokens`` and the graph-capture guard :496-515,
``combine`` :682-751, ``expand`` :753-873, ``aggregate`` :875-918, config getters, ``capture``, ``get_comm_stream``),
``deep_ep/backends/direct/resources.py`` (slot life cycle, generation-checked handle) and ``deep_ep/buffer.py:8-16``.
The V1 layout is the rank layout of :class:`ElasticBuffer` (``do_expand=False``): one received row per (source rank,
token), ``recv_topk_idx`` holding local expert ids.  ``get_dispatch_layout`` is its own small kernel (``ep_layout``).
Internode and the V1 low-latency entry points belong to multi-node RDMA deployments and raise
``NotImplementedError``; decode-size batches use ``ElasticBuffer``'s low-latency path.
"""
from __future__ import annotations

from typing import Optional

import torch

from ._compat import BUFFER_DISPATCH_ALIASES, BUFFER_INIT_ALIASES, SET_UNITS_ALIASES, keyword_aliases
from .config import Config
from .parallel.elastic import ElasticBuffer
from .parallel.streams import get_global_comm_stream
from .resources import Handle, SlotPool, SlotState
from .utils.event import EventHandle, EventOverlap

topk_idx_t = torch.int64


class Buffer:
    num_sms: int = 20

    def __init__(self, group, num_nvl_bytes: int = 0, num_rdma_bytes: int = 0, low_latency_mode: bool = False,
                 num_qps_per_rank: int = 24, allow_nvlink_for_low_latency_mode: bool = True, allow_mnnvl: bool = False,
                 explicitly_destroy: bool = False, enable_shrink: bool = False, comm=None, *, machine_type="auto",
                 rootinfo_path=None, hidden: int = 0, num_topk: int = 0, num_max_tokens_per_rank: int = 0, comm_stream=None):
        del num_qps_per_rank, allow_nvlink_for_low_latency_mode, allow_mnnvl, comm, machine_type, rootinfo_path
        if num_rdma_bytes:
            raise NotImplementedError("internode (RDMA) buffers are outside this single-NVLink-domain library")
        if low_latency_mode:
            raise NotImplementedError("use ElasticBuffer with num_max_tokens_per_rank <= 256 for low-latency decode")
        if enable_shrink:
            raise NotImplementedError("rank shrinking is not supported")
        self.group, self.num_nvl_bytes, self.explicitly_destroy = group, num_nvl_bytes, explicitly_destroy
        self._shape = (num_max_tokens_per_rank, hidden, num_topk)
        self._comm_stream = comm_stream                     # None: a stream of its own; "global": the process-wide one
        self._elastic: Optional[ElasticBuffer] = None
        self._slots = SlotPool()
        if all(self._shape):
            self._ensure(*self._shape)

    def _ensure(self, tokens: int, hidden: int, topk: int) -> ElasticBuffer:
        """V1 sizes its buffer in bytes only; the workspace is created on first use from the tensors' shape."""
        if self._elastic is None:
            if self.group is not None and not all(self._shape):
                # sized on first use: the ranks' batches may differ, the workspace may not, so they agree on the largest
                from .parallel.runtime import ControlPlane

                tokens = max(ControlPlane(self.group).all_gather_object(int(tokens)))
            self._elastic = ElasticBuffer(self.group, num_max_tokens_per_rank=max(tokens, 1), hidden=hidden, num_topk=topk,
                                          explicitly_destroy=self.explicitly_destroy, comm_stream=self._comm_stream)
        eb = self._elastic
        if tokens > eb.num_max_tokens_per_rank or hidden != eb.hidden or topk != eb.num_topk:
            raise ValueError("this Buffer was created for another (tokens, hidden, top-k) shape")
        return eb

    @property
    def machine_type(self) -> Optional[str]:
        """What the ranks run on (``None`` until the workspace exists); see ``ElasticBuffer.machine_type``."""
        return None if self._elastic is None else self._elastic.machine_type

    @property
    def machine_selection(self) -> Optional[dict]:
        return None if self._elastic is None else self._elastic.machine_selection

    # ------------------------------------------------------------------ resources
    def destroy(self) -> None:
        if self._elastic is not None:
            self._elastic.destroy()

    @staticmethod
    def set_num_sms(new_num_sms: int) -> None:
        if new_num_sms <= 0 or new_num_sms % 2:
            raise ValueError("the SM count must be a positive even number")
        Buffer.num_sms = new_num_sms

    set_num_compute_units = set_num_sms

    @staticmethod
    def capture() -> EventOverlap:
        return EventOverlap(EventHandle())

    def get_comm_stream(self):
        return None if self._elastic is None else self._elastic.get_comm_stream()

    @staticmethod
    def get_dispatch_config(num_ranks: int) -> Config:
        return Config(Buffer.num_sms, 6, 256, 6, 128)

    @staticmethod
    def get_combine_config(num_ranks: int) -> Config:
        return Config(Buffer.num_sms, 4, 256, 6, 128)

    @staticmethod
    def get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank, hidden, num_ranks, num_experts) -> int:
        from .parallel import layout as L

        del num_experts
        return L.elastic_size_hint(num_ranks, num_max_dispatch_tokens_per_rank, hidden, 8)

    get_low_latency_scaleout_size_hint = get_low_latency_rdma_size_hint

    # ------------------------------------------------------------------ V1 operations
    def get_dispatch_layout(self, topk_idx: torch.Tensor, num_experts: int, previous_event=None, async_finish: bool = False,
                            allocate_on_comm_stream: bool = False):
        """(num_tokens_per_rank, num_tokens_per_rdma_rank=None, num_tokens_per_expert, is_token_in_rank, event).

        On a GPU this is the ``ep_layout`` kernel; on CPU tensors the same counts in torch."""
        del allocate_on_comm_stream
        world = 1 if self.group is None else torch.distributed.get_world_size(self.group)
        if topk_idx.dim() != 2 or topk_idx.dtype != torch.int64 or not topk_idx.is_contiguous():
            raise ValueError("topk_idx must be contiguous int64 [tokens, top-k]")
        if num_experts <= 0 or num_experts % world or num_experts > 1024:
            raise ValueError("num_experts must be a positive multiple of the world size, at most 1024")
        if previous_event is not None and getattr(previous_event, "event", None) is not None:
            previous_event.current_stream_wait()
        T, K = topk_idx.shape
        if topk_idx.is_cuda:
            from .ops import require_native

            C = require_native("Buffer.get_dispatch_layout")
            dev = topk_idx.device
            per_rank = torch.zeros((world,), dtype=torch.int32, device=dev)
            per_expert = torch.zeros((num_experts,), dtype=torch.int32, device=dev)
            in_rank = torch.empty((T, world), dtype=torch.bool, device=dev)
            C.layout(topk_idx.data_ptr(), T, K, num_experts, world, per_rank.data_ptr(), per_expert.data_ptr(), in_rank.data_ptr(),
                     torch.cuda.current_stream(dev).cuda_stream)
            event = EventOverlap._from_resources(EventHandle(), (per_rank, per_expert, in_rank, topk_idx)) if async_finish \
                else EventOverlap()
            return per_rank, None, per_expert, in_rank, event
        local = num_experts // world
        valid = (topk_idx >= 0) & (topk_idx < num_experts)
        dst = torch.where(valid, torch.div(topk_idx, local, rounding_mode="floor"), torch.full_like(topk_idx, -1))
        in_rank = torch.stack([(dst == r).any(dim=1) for r in range(world)], dim=1)
        per_expert = torch.bincount(topk_idx[valid], minlength=num_experts).to(torch.int32)
        return in_rank.sum(0).to(torch.int32), None, per_expert, in_rank, EventOverlap()

    def _v1_handle(self, eh, in_rank: Optional[torch.Tensor], tokens: int) -> Handle:
        """Upstream's six handle tensors from the routing plan of the dispatch, bound to a slot."""
        plan = eh._plan
        tmax, K = self._elastic.num_max_tokens_per_rank, self._elastic.num_topk
        rank_prefix = torch.cumsum(plan.rank_matrix.to(torch.int64), dim=0).to(torch.int32)
        recv_src_idx = (torch.div(plan.recv_row_src[:plan.num_rows], K, rounding_mode="floor") % tmax).to(torch.int32)
        send_head = plan.send_slot[:tokens]
        if in_rank is None:
            in_rank = send_head >= 0
        slot = self._slots.acquire()
        slot.move(SlotState.DISPATCH_IN_FLIGHT)
        slot.move(SlotState.DISPATCH_READY)
        return Handle((rank_prefix, plan.send_chunk_prefix, plan.chunk_start, recv_src_idx, in_rank, send_head), slot, eh)

    def dispatch(self, x, handle=None, num_tokens_per_rank=None, num_tokens_per_rdma_rank=None, is_token_in_rank=None,
                 num_tokens_per_expert=None, topk_idx=None, topk_weights=None, expert_alignment: int = 1, num_worst_tokens: int = 0,
                 config: Optional[Config] = None, previous_event=None, async_finish: bool = False,
                 allocate_on_comm_stream: bool = False, zero_copy: bool = False):
        """(recv_x, recv_topk_idx, recv_topk_weights, num_recv_tokens_per_expert_list, handle, event).

        ``expert_alignment`` rounds the per-expert counts of the returned list up (the rows themselves keep the rank
        layout).  ``num_worst_tokens > 0`` gives outputs of exactly that many rows without any host synchronisation
        (the list is empty then); it must equal ``group size x num_max_tokens_per_rank`` and is required while the
        current stream is being captured into a CUDA graph.  ``zero_copy`` (the reference's extension,
        ``deep_ep/backends/direct/buffer.py:481-496``: outputs may alias the workspace) is accepted; the outputs here
        always own their storage, which satisfies either setting."""
        del num_tokens_per_rank, num_tokens_per_rdma_rank
        if not isinstance(zero_copy, bool):
            raise TypeError("zero_copy must be a bool")
        if expert_alignment < 1:
            raise ValueError("expert_alignment must be positive")
        data = x[0] if isinstance(x, (tuple, list)) else x
        sms = config.num_sms if config is not None else 0
        capturing = data.is_cuda and torch.cuda.is_current_stream_capturing()
        if handle is not None:
            if not isinstance(handle, Handle):
                raise TypeError("handle must come from Buffer.dispatch")
            handle.check_live()
            eb = self._ensure(data.shape[0], data.shape[1], handle.topk_idx.shape[1])
            handle.slot.move(SlotState.DISPATCH_IN_FLIGHT)
            rx, _, _, _, ev = eb.dispatch(x, handle=handle.elastic, num_sms=sms, previous_event=previous_event,
                                          async_with_compute_stream=async_finish, allocate_on_comm_stream=allocate_on_comm_stream)
            handle.slot.move(SlotState.DISPATCH_READY)
            return rx, None, None, None, handle, ev
        if topk_idx is None or num_tokens_per_expert is None:
            raise ValueError("a fresh V1 dispatch needs topk_idx and num_tokens_per_expert (from get_dispatch_layout)")
        eb = self._ensure(data.shape[0], data.shape[1], topk_idx.shape[1])
        if capturing and num_worst_tokens == 0:
            raise RuntimeError("a fresh dispatch inside a CUDA graph capture cannot read the row count back: pass num_worst_tokens")
        if num_worst_tokens and num_worst_tokens != eb.world_size * eb.num_max_tokens_per_rank:
            raise ValueError(f"num_worst_tokens must be group size x num_max_tokens_per_rank = "
                             f"{eb.world_size * eb.num_max_tokens_per_rank}")
        rx, ridx, rw, h, ev = eb.dispatch(x, topk_idx=topk_idx, topk_weights=topk_weights, num_experts=num_tokens_per_expert.numel(),
                                          num_sms=sms, previous_event=previous_event, async_with_compute_stream=async_finish,
                                          allocate_on_comm_stream=allocate_on_comm_stream, do_expand=False,
                                          do_cpu_sync=(num_worst_tokens == 0), num_max_tokens_per_rank=10 ** 9, _rank_matrix=True)
        counts = h.num_recv_tokens_per_expert_list
        if counts is not None and expert_alignment > 1:
            counts = [-(-c // expert_alignment) * expert_alignment for c in counts]
        return rx, ridx, rw, ([] if counts is None else counts), self._v1_handle(h, is_token_in_rank, data.shape[0]), ev

    def combine(self, x, handle, topk_weights=None, bias=None, config: Optional[Config] = None, previous_event=None,
                async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """(combined_x, combined_topk_weights, event)."""
        if self._elastic is None:
            raise RuntimeError("combine needs the buffer that produced the handle")
        if not isinstance(handle, Handle):
            raise TypeError("handle must come from Buffer.dispatch")
        handle.check_live()
        handle.slot.move(SlotState.COMBINE_IN_FLIGHT)
        try:
            out = self._elastic.combine(x, handle.elastic, topk_weights=topk_weights, bias=bias,
                                        num_sms=config.num_sms if config else 0, previous_event=previous_event,
                                        async_with_compute_stream=async_finish, allocate_on_comm_stream=allocate_on_comm_stream)
        except Exception:
            handle.slot.move(SlotState.DISPATCH_READY)
            raise
        handle.slot.move(SlotState.RELEASABLE)       # still usable (backward passes) until a later dispatch needs the slot
        return out

    def release(self, handle: Handle) -> None:
        """Give the handle's slot back now instead of waiting for a later dispatch to recycle it."""
        if isinstance(handle, Handle) and handle.slot is not None and handle.slot.generation == handle.generation:
            self._slots.release(handle.slot)

    def _ordered(self, fn, previous_event, async_finish: bool, tensors):
        """Runs a local operator on the current stream after ``previous_event``; returns its results and an event."""
        if previous_event is not None and getattr(previous_event, "event", None) is not None:
            previous_event.current_stream_wait()
        result = fn()
        if async_finish and torch.cuda.is_available() and tensors(result) and tensors(result)[0].is_cuda:
            return result, EventOverlap._from_resources(EventHandle(), tuple(t for t in tensors(result) if t is not None))
        return result, EventOverlap()

    def expand(self, x, recv_topk_idx=None, topk_weights=None, num_tokens_per_expert=None, expert_alignment=None, handle=None,
               config: Optional[Config] = None, previous_event=None, async_finish: bool = False,
               allocate_on_comm_stream: bool = False):
        """Expand rank-deduplicated dispatch rows into expert-major rows:
        ``(expanded_x | (expanded_x, scales), expanded_topk_weights, ExpandHandle, event)``."""
        from .ops.expand import expand as _expand

        del config, allocate_on_comm_stream
        (ex, ew, h), ev = self._ordered(lambda: _expand(x, recv_topk_idx, topk_weights, num_tokens_per_expert, expert_alignment, handle),
                                        previous_event, async_finish,
                                        lambda r: [*(r[0] if isinstance(r[0], tuple) else (r[0],)), r[1]])
        return ex, ew, h, ev

    def aggregate(self, x, handle, topk_weights=None, expanded_values=None, config: Optional[Config] = None, previous_event=None,
                  async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """Reduce expert-major rows back to the rank-deduplicated layout: ``(aggregated_x, aggregated_values, event)``."""
        from .ops.expand import aggregate as _aggregate

        del config, allocate_on_comm_stream
        (ax, av), ev = self._ordered(lambda: _aggregate(x, handle, topk_weights, expanded_values), previous_event, async_finish,
                                     lambda r: [r[0], r[1]])
        return ax, av, ev

    # ------------------------------------------------------------------ not part of this library
    def internode_dispatch(self, *a, **k): raise NotImplementedError("internode dispatch needs an RDMA fabric")
    def internode_combine(self, *a, **k): raise NotImplementedError("internode combine needs an RDMA fabric")
    def clean_low_latency_buffer(self, *a, **k): raise NotImplementedError("V1 low-latency mode: use ElasticBuffer")
    def low_latency_dispatch(self, *a, **k): raise NotImplementedError("V1 low-latency mode: use ElasticBuffer")
    def low_latency_combine(self, *a, **k): raise NotImplementedError("V1 low-latency mode: use ElasticBuffer")
    def get_next_low_latency_combine_buffer(self, *a, **k): raise NotImplementedError("V1 low-latency mode: use ElasticBuffer")


__all__ = ["Buffer", "Handle", "get_global_comm_stream", "topk_idx_t"]


# platform-neutral spellings next to the upstream ones (parity: ``deep_ep/backends/direct/api.py:8-20`` of the reference)
Buffer.__init__ = keyword_aliases(Buffer.__init__, BUFFER_INIT_ALIASES)
Buffer.dispatch = keyword_aliases(Buffer.dispatch, BUFFER_DISPATCH_ALIASES)
Buffer.set_num_sms = staticmethod(keyword_aliases(Buffer.__dict__["set_num_sms"].__func__, SET_UNITS_ALIASES))
Buffer.set_num_compute_units = Buffer.__dict__["set_num_sms"]
