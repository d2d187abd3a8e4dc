"""CUDA engine: drives the native kernels for one rank, or for several virtual ranks on one GPU.

All methods take *lists* with one entry per rank handled by this process.  A
production ``ElasticBuffer`` passes one-element lists; :class:`VirtualWorld`
passes one entry per virtual rank so the whole cross-rank protocol runs inside
one cooperative launch on a single GPU.

Parity: host op wrappers ``csrc/ops/{notify,dispatch,combine}.cpp`` of the
reference (argument validation, tiling, launch); the count read-back is the
single host synchronisation of a fresh dispatch
(``deep_ep/backends/mesh_clos/elastic.py:1473-1479``).
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
import os
from typing import List, Optional, Sequence, Tuple

import torch

from ..ops import require_native

STATUS_NAMES = {0: "ok", 1: "timeout", 2: "bad argument", 3: "aborted"}
OP_NAMES = {0: "barrier", 1: "notify", 2: "dispatch", 3: "combine", 4: "ll_dispatch", 5: "ll_combine", 6: "mega_moe",
            7: "alltoallv_gmm", 8: "gmm_alltoallv"}
# what a kernel was waiting for at each wait site (operation, site) when its time limit ran out; sites of 100 and above are
# index checks of the index-checking build
WAIT_SITES = {
    (0, 0): "the peer to reach the barrier", (0, 99): "a flag that nothing sets (the wait probe of the tests)",
    (1, 0): "the peer to finish reading the previous routing tables", (1, 1): "the peer's routing table",
    (2, 0): "the peer to finish the previous dispatch", (2, 1): "rows of a source rank to land in the staging area",
    (3, 0): "the peer to finish the previous combine", (3, 1): "the partial sums of an expert rank",
    (4, 0): "the peer to release the bank used two calls ago", (4, 1): "the peer's routing table", (4, 2): "a part of a row from a source rank",
    (5, 0): "the peer to release the bank used two calls ago", (5, 1): "a part of an expert's row",
    (6, 0): "the peer's inputs and routing table", (6, 1): "the peer's combine rows",
    (7, 0): "the peer to finish the previous call", (7, 1): "the peer's staged rows and row table",
    (8, 0): "the peer's row table", (8, 1): "the rows returned by the peer",
}


class CommunicationError(RuntimeError):
    pass


@dataclass
class RoutingPlan:
    """Device-side routing metadata of one dispatch (what an ``EPHandle`` owns)."""
    num_tokens: int
    num_experts: int
    num_topk: int
    expand: bool
    alignment: int
    meta_stride: int
    num_rows: int                       # output rows (exact, or the worst case without a host sync)
    num_staged_rows: int
    expert_counts_list: Optional[List[int]]
    topk_idx: torch.Tensor
    send_slot: Optional[torch.Tensor]
    slot_row: Optional[torch.Tensor]
    stage_meta: Optional[torch.Tensor]
    chunk_start: Optional[torch.Tensor]
    rank_tokens: Optional[torch.Tensor]
    rank_rows: Optional[torch.Tensor]
    expert_counts: torch.Tensor
    expert_offsets: torch.Tensor
    recv_row_src: torch.Tensor
    recv_w: Optional[torch.Tensor]
    recv_idx: Optional[torch.Tensor]
    has_weights: bool = False
    low_latency: bool = False
    num_rows_dev: Optional[torch.Tensor] = None
    topk_w: Optional[torch.Tensor] = None
    rank_matrix: Optional[torch.Tensor] = None
    send_chunk_prefix: Optional[torch.Tensor] = None

    def tensors(self):
        return [t for t in (self.topk_idx, self.send_slot, self.slot_row, self.stage_meta, self.chunk_start, self.rank_tokens,
                            self.rank_rows, self.expert_counts, self.expert_offsets, self.recv_row_src, self.recv_w,
                            self.recv_idx) if t is not None]


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


# Share of the blocks on the side that drives NVLink (dispatch: senders, combine: expert side), by world size.
DISPATCH_SEND_FRACTION = {1: 1.0, 2: 0.5, 4: 0.35, 8: 0.35}
COMBINE_SEND_FRACTION = {1: 0.0, 2: 0.5, 4: 0.6, 8: 0.6}


class CudaEngine:
    def __init__(self, sessions: Sequence, layout, device: torch.device, num_sms: int = 0, host_timeout: float = 300.0):
        self.C = require_native("ElasticBuffer")
        self.host_timeout = float(host_timeout)       # limit of the host's waits for a kernel whose results it reads back
        self.sessions = list(sessions)
        self.layout = layout
        self.device = device
        self.n = len(self.sessions)
        self.world = layout.world
        props = torch.cuda.get_device_properties(device)
        self.sm_count = props.multi_processor_count
        per_rank = max(2, self.sm_count // self.n)
        # One block per SM.  The sender side of dispatch (expert side of combine) has to keep NVLink busy, which takes
        # 32 SMs or more; the other side moves the rows inside local memory.  With one rank every row is local and is
        # written (read) directly by the sender (source) side, so that side gets all the blocks.
        budget = min(per_rank, num_sms) if num_sms else min(per_rank, max(2, self.sm_count - 4))
        self.dispatch_blocks = self.combine_blocks = self.default_blocks = budget
        self.dispatch_send_fraction = DISPATCH_SEND_FRACTION.get(self.world, 0.35)
        self.combine_send_fraction = COMBINE_SEND_FRACTION.get(self.world, 0.6)
        # rows that stay on their rank bypass the staging area / the partial area (see the kernels' headers)
        self.local_direct = os.environ.get("DEEPEP_HT_LOCAL_DIRECT", "1") not in ("", "0")
        nt = -(-layout.max_tokens // self.C.chunk_tokens)
        self._nt = nt
        # opt-in device timing of every launch (DEEPEP_PROFILE=1 or enable_profiling()): events around each kernel
        self._profile = os.environ.get("DEEPEP_PROFILE", "0") not in ("", "0")
        self._timings: List[Tuple[str, "torch.cuda.Event", "torch.cuda.Event"]] = []
        # opt-in device-side records (the profile instantiation of the dispatch / combine kernels): one record per block
        self._device_profile = False
        self._prof: dict = {}
        self._scratch = []
        for _ in range(self.n):
            self._scratch.append(dict(
                hist=torch.empty((self.world * nt * self.C.max_experts,), dtype=torch.int32, device=device),
                hits=torch.empty((self.world * nt,), dtype=torch.int32, device=device),
                own_hits=torch.empty((nt * self.world,), dtype=torch.int32, device=device),
                cnt=torch.empty((self.world * self.C.max_experts,), dtype=torch.int32, device=device)))

    # ------------------------------------------------------------------ helpers
    def _stream(self, stream=None) -> int:
        """Launch stream: ``stream`` if given, else the current stream.  Tensors are always allocated on the
        *current* stream, so a caller that launches on a side stream and then makes the current stream wait for it
        needs no ``record_stream`` bookkeeping."""
        return (stream if stream is not None else torch.cuda.current_stream(self.device)).cuda_stream

    # ------------------------------------------------------------------ device phase timing
    def enable_profiling(self, on: bool = True) -> None:
        """Record a pair of CUDA events around every kernel launch (parity: the reference's ``DevicePhaseTiming``,
        ``csrc/ops/device_phase_timing.hpp:13-50``, and the optional event timing of its notify op)."""
        self._profile = bool(on)
        self._timings.clear()

    def enable_device_profile(self, on: bool = True) -> None:
        """Launch the profile instantiation of the kernels (``template <bool kProfile>``).  Notify and the low-latency
        kernels stamp the phases of their block 0 (read with ``phase_stamps``); in the high-throughput dispatch /
        combine every block records its role, its start and end time, the time its first warp spent waiting for
        flags and the rows that warp moved.  The production instantiation carries none of that code.
        Parity: the reference's ``template <bool Profile>`` kernels (``csrc/kernels/dispatch/profile.hpp``,
        ``csrc/kernels/combine/profile.hpp``)."""
        self._device_profile = bool(on)
        self._prof.clear()

    PHASE_STAMPS = {"ll_dispatch": (0, ("routes_read", "rows_sent", "tables_in", "layout_done", "rows_out", "last_block", "table_sent",
                                        "first_row_stored")),
                    "ll_combine": (8, ("entered", "rows_returned", "reduced", "last_block")),
                    "notify": (16, ("table_sent", "tables_in", "histograms", "scans", "records", "done"))}

    def phase_stamps(self, op: str, i: int = 0) -> dict:
        """Phase stamps of block 0 of the last profiled launch of ``op`` (``"notify"``, ``"ll_dispatch"`` or
        ``"ll_combine"``) on rank index ``i``: microseconds since the kernel started at which each phase was complete.
        Only the profile instantiations of these kernels write stamps (``enable_device_profile``)."""
        first, names = self.PHASE_STAMPS[op]
        torch.cuda.synchronize(self.device)
        words = torch.frombuffer(bytearray(self.sessions[i].read_control()), dtype=torch.int64)
        at = self.C.control_dbg_offset // 8 + first
        return {name: int(words[at + k]) / 1e3 for k, name in enumerate(names)}

    def _prof_buffer(self, op: str, i: int):
        if not self._device_profile:
            return None
        words = self.C.dispatch_prof_words if op == "dispatch" else self.C.combine_prof_words
        key = (op, i)
        if key not in self._prof:
            self._prof[key] = torch.zeros((self.sm_count, words), dtype=torch.int64, device=self.device)
        return self._prof[key].data_ptr()

    def pop_device_profile(self) -> dict:
        """``{(op, rank index): [per-block dict]}`` of the last profiled launch of each op: ``role``, ``start_us`` /
        ``end_us`` (relative to the earliest block start of the launch), and, averaged over the block's warps, the
        microseconds spent reading routing records (``meta_us``), waiting for flags (``wait_us``), moving or reducing
        rows (``data_us``) and publishing flags (``publish_us``); ``rows`` counts the rows the block handled."""
        torch.cuda.synchronize(self.device)
        mhz = torch.cuda.get_device_properties(self.device).clock_rate / 1e3 if hasattr(
            torch.cuda.get_device_properties(self.device), "clock_rate") else 1965.0
        out = {}
        for key, buf in self._prof.items():
            warps = (self.C.dispatch_threads if key[0] == "dispatch" else self.C.combine_threads) / 32.0
            rows = [r for r in buf.cpu().tolist() if r[2] > 0]
            if not rows:
                continue
            t0 = min(r[1] for r in rows)
            side = ("sender", "receiver") if key[0] == "dispatch" else ("expert", "source")
            out[key] = [dict(role=side[int(r[0])], start_us=(r[1] - t0) / 1e3, end_us=(r[2] - t0) / 1e3,
                             meta_us=r[3] / mhz / warps, wait_us=r[4] / mhz / warps, data_us=r[5] / mhz / warps,
                             publish_us=r[6] / mhz / warps, rows=int(r[7])) for r in rows]
            buf.zero_()
        return out

    def _timed(self, name: str, stream, launch) -> None:
        if not self._profile:
            launch()
            return
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(st)
        launch()
        end.record(st)
        self._timings.append((name, start, end))
        if len(self._timings) > 4096:
            del self._timings[:2048]

    def pop_timings(self) -> List[Tuple[str, float]]:
        """``[(kernel, microseconds)]`` of the launches recorded so far (synchronises on their end events)."""
        out = []
        for name, start, end in self._timings:
            end.synchronize()
            out.append((name, start.elapsed_time(end) * 1e3))
        self._timings.clear()
        return out

    def _host_wait(self, stream, what: str) -> None:
        """The host needs the results of what was just queued on ``stream``: wait for it, but not for ever."""
        from ..utils.hostwait import HostTimeout, wait_for_event

        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        done = torch.cuda.Event()
        done.record(st)
        try:
            wait_for_event(done, self.host_timeout, what)
        except HostTimeout as exc:
            raise CommunicationError(f"{exc}; restart the distributed job") from None
        st.synchronize()                               # returns at once: everything before the event is complete

    def check_status(self) -> None:
        for s in self.sessions:
            st = s.status()
            if st["code"] != 0:
                what = WAIT_SITES.get((st["op"], st["where"]))
                raise CommunicationError(
                    f"rank {st['rank']}: {OP_NAMES.get(st['op'], st['op'])} {STATUS_NAMES.get(st['code'], st['code'])} "
                    f"at wait site {st['where']}" + (f" ({what})" if what else "") + f" on peer {st['peer']} "
                    f"(expected {st['expected']}, saw {st['seen']}); restart the distributed job")

    def split_blocks(self, total: int, send_fraction: float, default: int = 0) -> Tuple[int, int]:
        """(blocks of the NVLink side, blocks of the local side).  A fraction of 1.0 / 0.0 gives every block to one
        side, which only a single rank with direct local rows may do."""
        total = max(2, min(total, self.sm_count // self.n) if total else (default or self.default_blocks))
        if self.world == 1 and self.local_direct and send_fraction in (0.0, 1.0):
            return (total, 0) if send_fraction == 1.0 else (0, total)
        send = min(total - 1, max(1, int(round(total * send_fraction))))
        return send, total - send

    def row_capacity(self, num_experts: int, alignment: int, expand: bool) -> int:
        local = num_experts // self.world
        k = self.layout.topk
        per_token = min(k, local) if expand else 1
        cap = self.world * self.layout.max_tokens * per_token
        if expand and alignment > 1:
            cap += local * (alignment - 1)
        return cap

    # ------------------------------------------------------------------ ops
    def notify(self, topk_idx: Sequence[torch.Tensor], topk_w: Sequence[Optional[torch.Tensor]], num_experts: int,
               expand: bool = True, alignment: int = 1, cpu_sync: bool = True, blocks: int = 0, stream=None,
               rank_matrix: bool = False) -> List[RoutingPlan]:
        """``rank_matrix``: also count, on every rank, the tokens each source sends to each rank (``plan.rank_matrix
        [P, P]``, what the V1 handle's ``rank_prefix_matrix`` is built from) and keep this rank's per-chunk send
        prefixes (``plan.send_chunk_prefix [P, chunks]``)."""
        C, lay, dev = self.C, self.layout, self.device
        P, K = self.world, lay.topk
        local = num_experts // P
        stride = 2 + max(2, min(K, local))
        rcap = self.row_capacity(num_experts, alignment, expand)
        plans, args = [], []
        for i in range(self.n):
            idx = topk_idx[i]
            T = idx.shape[0]
            i32 = dict(dtype=torch.int32, device=dev)
            plan = RoutingPlan(
                num_tokens=T, num_experts=num_experts, num_topk=K, expand=expand, alignment=alignment, meta_stride=stride,
                num_rows=rcap, num_staged_rows=0, expert_counts_list=None, topk_idx=idx,
                send_slot=torch.empty((max(T, 1), P), **i32), slot_row=torch.empty((max(T, 1), K), **i32),
                stage_meta=torch.empty((P * lay.max_tokens, stride), **i32),
                chunk_start=torch.empty((P, self._nt + 1), **i32), rank_tokens=torch.empty((P,), **i32),
                rank_rows=torch.empty((P + 1,), **i32), expert_counts=torch.empty((local,), **i32),
                expert_offsets=torch.empty((local + 1,), **i32), recv_row_src=torch.empty((rcap,), **i32),
                recv_w=(torch.empty((rcap,) if expand else (rcap, K), dtype=torch.float32, device=dev)
                        if topk_w[i] is not None else None),
                recv_idx=None if expand else torch.empty((rcap, K), dtype=torch.int64, device=dev),
                has_weights=topk_w[i] is not None)
            plan.rank_matrix = torch.zeros((P, P), **i32) if rank_matrix else None
            plans.append(plan)
            sc = self._scratch[i]
            args.append(dict(topk_idx=idx.data_ptr(), topk_w=_ptr(topk_w[i]), T=T, E=num_experts, K=K, expand=int(expand),
                             alignment=alignment, meta_stride=stride, hist=sc["hist"].data_ptr(), hits=sc["hits"].data_ptr(),
                             own_hits=sc["own_hits"].data_ptr(), cnt=sc["cnt"].data_ptr(), send_slot=plan.send_slot.data_ptr(),
                             slot_row=plan.slot_row.data_ptr(), stage_meta=plan.stage_meta.data_ptr(),
                             chunk_start=plan.chunk_start.data_ptr(), rank_tokens=plan.rank_tokens.data_ptr(),
                             rank_rows=plan.rank_rows.data_ptr(), expert_counts=plan.expert_counts.data_ptr(),
                             expert_offsets=plan.expert_offsets.data_ptr(), recv_row_src=plan.recv_row_src.data_ptr(),
                             recv_w=_ptr(plan.recv_w), recv_idx=_ptr(plan.recv_idx), rcap=rcap,
                             rank_matrix=_ptr(plan.rank_matrix)))
        # the layout pass is a chain of short phases over (source, tile) tasks: P x T / 64 of them, a few microseconds each
        nblocks = blocks or max(1, min(128, self.sm_count // self.n))
        self._timed("notify", stream, lambda: C.notify(lay, self.sessions, args, nblocks, self._stream(stream), self._device_profile))
        if rank_matrix:       # the scratch is reused by the next call: keep this rank's per-chunk send prefixes with the plan
            for plan, sc in zip(plans, self._scratch):
                tiles = -(-max(plan.num_tokens, 1) // C.chunk_tokens)
                with torch.cuda.stream(stream) if stream is not None else contextlib.nullcontext():
                    plan.send_chunk_prefix = sc["own_hits"][:tiles * P].view(tiles, P).t().contiguous()
        if cpu_sync:
            self._host_wait(stream, "the routing layout pass")
            self.check_status()
            for plan, s in zip(plans, self.sessions):
                box = s.mailbox(4 + local)
                if box[0] < 0:
                    raise CommunicationError("notify did not complete; restart the distributed job")
                plan.num_rows, plan.num_staged_rows = box[0], box[1]
                plan.expert_counts_list = box[4:4 + local]
        return plans

    def dispatch(self, xs: Sequence, plans: Sequence[RoutingPlan], mode: int, blocks: int = 0, stream=None,
                 split: Optional[Tuple[int, int]] = None):
        """xs[i] is a tensor (modes 0, 2) or a (fp8, scales) pair (mode 1). Returns [(recv_x, recv_sf | None)].
        ``split`` = (sender blocks, receiver blocks) overrides the default division."""
        lay, dev = self.layout, self.device
        H = lay.hidden
        outs, args = [], []
        for i, plan in enumerate(plans):
            x, sf = (xs[i] if isinstance(xs[i], (tuple, list)) else (xs[i], None))
            rows = plan.num_rows
            if mode == 0:
                recv_x = torch.empty((rows, H), dtype=x.dtype, device=dev)
                recv_sf = None
            else:
                recv_x = torch.empty((rows, H), dtype=torch.float8_e4m3fn, device=dev)
                recv_sf = torch.empty((rows, H // 128), dtype=torch.float32, device=dev)
            if plan.expand and plan.alignment > 1:
                recv_x.view(torch.uint8).zero_()
                if recv_sf is not None:
                    recv_sf.zero_()
            outs.append((recv_x, recv_sf))
            args.append(dict(x=x.data_ptr(), x_sf=_ptr(sf), T=plan.num_tokens, mode=mode, send_slot=plan.send_slot.data_ptr(),
                             slot_row=plan.slot_row.data_ptr(), topk_idx=plan.topk_idx.data_ptr(),
                             stage_meta=plan.stage_meta.data_ptr(),
                             rank_tokens=plan.rank_tokens.data_ptr(), rank_rows=plan.rank_rows.data_ptr(),
                             meta_stride=plan.meta_stride, K=plan.num_topk, E=plan.num_experts, expand=int(plan.expand),
                             recv_x=recv_x.data_ptr(), recv_sf=_ptr(recv_sf), recv_rows=recv_x.shape[0],
                             prof=self._prof_buffer("dispatch", i)))
        send, recv = split if split is not None else self.split_blocks(blocks, self.dispatch_send_fraction, self.dispatch_blocks)
        self._timed("dispatch", stream, lambda: self.C.dispatch(lay, self.sessions, args, send, recv, self._stream(stream),
                                                                self.local_direct, self._device_profile))
        return outs

    def combine(self, xs: Sequence[torch.Tensor], plans: Sequence[RoutingPlan], ws: Sequence[Optional[torch.Tensor]],
                bias: Sequence = None, blocks: int = 0, stream=None, split: Optional[Tuple[int, int]] = None):
        """``split`` = (expert-side sender blocks, source-side reducer blocks) overrides the default division."""
        lay, dev = self.layout, self.device
        H, K = lay.hidden, lay.topk
        outs, args = [], []
        for i, plan in enumerate(plans):
            T = plan.num_tokens
            out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
            out_w = torch.empty((T, K), dtype=torch.float32, device=dev) if ws[i] is not None else None
            b = bias[i] if bias is not None else None
            b0, b1 = (b if isinstance(b, (tuple, list)) else (b, None)) if b is not None else (None, None)
            outs.append((out, out_w))
            args.append(dict(x=xs[i].data_ptr(), w=_ptr(ws[i]), stage_meta=plan.stage_meta.data_ptr(),
                             rank_rows=plan.rank_rows.data_ptr(), rank_tokens=plan.rank_tokens.data_ptr(),
                             prof=self._prof_buffer("combine", i),
                             send_slot=plan.send_slot.data_ptr(), topk_idx=plan.topk_idx.data_ptr(), T=T,
                             meta_stride=plan.meta_stride, K=K, E=plan.num_experts, expand=int(plan.expand),
                             bias0=_ptr(b0), bias1=_ptr(b1), out=out.data_ptr(), out_w=_ptr(out_w), x_rows=xs[i].shape[0]))
        send, recv = self.split_blocks(blocks, self.combine_send_fraction, self.combine_blocks)
        if split is not None:
            limit = max(2, self.sm_count // self.n)
            send, recv = max(1, int(split[0])), max(1, int(split[1]))
            if send + recv > limit:
                raise ValueError(f"combine_num_sms + reduce_num_sms must not exceed {limit} on this device")
        # one launch per token window: all tokens at once unless the workspace holds the partials of fewer tokens
        window, most = lay.partial_tokens, max([plan.num_tokens for plan in plans] + [1])
        if self.n == 1 and self.world > 1 and window < lay.max_tokens:
            most = lay.max_tokens         # real ranks cannot see each other's token counts: every rank runs every pass
        for begin in range(0, most, window):
            self._timed("combine", stream, lambda b=begin: self.C.combine(lay, self.sessions, args, send, recv, self._stream(stream),
                                                                          self.local_direct, self._device_profile, b, b + window))
        return outs

    # ------------------------------------------------------------------ low latency
    def ll_blocks(self) -> int:
        return max(1, min(128, self.sm_count // self.n))   # at most a part of a row or two per warp: latency is the goal

    def ll_dispatch(self, xs: Sequence, topk_idx: Sequence[torch.Tensor], topk_w: Sequence[torch.Tensor], num_experts: int,
                    mode: int, cpu_sync: bool = True, stream=None, outputs: Optional[list] = None):
        """One kernel: routing exchange + row push + expert-major receive.  Returns [(plan, recv_x, recv_sf | None)].

        Outputs have the worst-case row count; with ``cpu_sync`` they are trimmed to the exact count after one
        host synchronisation.  ``outputs`` lets a caller supply pre-allocated buffers (CUDA-graph capture).
        """
        lay, dev = self.layout, self.device
        P, K, H = self.world, lay.topk, lay.hidden
        local = num_experts // P
        cap = P * lay.max_tokens * min(K, local)
        res, args = [], []
        for i in range(self.n):
            x, sf = (xs[i] if isinstance(xs[i], (tuple, list)) else (xs[i], None))
            T = x.shape[0]
            i32 = dict(dtype=torch.int32, device=dev)
            if outputs is not None:
                o = outputs[i]
            else:
                o = dict(recv_x=torch.empty((cap, H), dtype=x.dtype if mode == 0 else torch.float8_e4m3fn, device=dev),
                         recv_sf=None if mode == 0 else torch.empty((cap, H // 128), dtype=torch.float32, device=dev),
                         recv_w=torch.empty((cap,), dtype=torch.float32, device=dev),
                         recv_row_src=torch.empty((cap,), **i32), expert_counts=torch.empty((local,), **i32),
                         expert_offsets=torch.empty((local + 1,), **i32), num_rows=torch.empty((1,), **i32))
            plan = RoutingPlan(num_tokens=T, num_experts=num_experts, num_topk=K, expand=True, alignment=1, meta_stride=0,
                               num_rows=cap, num_staged_rows=0, expert_counts_list=None, topk_idx=topk_idx[i], send_slot=None,
                               slot_row=None, stage_meta=None, chunk_start=None, rank_tokens=None, rank_rows=None,
                               expert_counts=o["expert_counts"], expert_offsets=o["expert_offsets"],
                               recv_row_src=o["recv_row_src"], recv_w=o["recv_w"], recv_idx=None, has_weights=True)
            plan.num_rows_dev, plan.topk_w, plan.low_latency = o["num_rows"], topk_w[i], True
            res.append((plan, o["recv_x"], o["recv_sf"]))
            args.append(dict(x=x.data_ptr(), x_sf=_ptr(sf), topk_idx=topk_idx[i].data_ptr(), topk_w=topk_w[i].data_ptr(), T=T,
                             E=num_experts, mode=mode, recv_x=o["recv_x"].data_ptr(), recv_sf=_ptr(o["recv_sf"]),
                             recv_w=o["recv_w"].data_ptr(), recv_row_src=o["recv_row_src"].data_ptr(),
                             expert_counts=o["expert_counts"].data_ptr(), expert_offsets=o["expert_offsets"].data_ptr(),
                             num_rows=o["num_rows"].data_ptr(), use_mailbox=int(cpu_sync), capacity=cap))
        self._timed("ll_dispatch", stream, lambda: self.C.ll_dispatch(lay, self.sessions, args, self.ll_blocks(), self._stream(stream),
                                                                             self._device_profile))
        if cpu_sync:
            self._host_wait(stream, "the low-latency dispatch")
            self.check_status()
            out = []
            for (plan, rx, rsf), s in zip(res, self.sessions):
                box = s.mailbox(4 + local)
                plan.num_rows, plan.expert_counts_list = box[0], box[4:4 + local]
                out.append((plan, rx[:box[0]], None if rsf is None else rsf[:box[0]]))
            return out
        return res

    def ll_dispatch_cached(self, xs: Sequence, plans: Sequence[RoutingPlan], mode: int, stream=None):
        """Re-run the self-contained low-latency dispatch with the routing saved in the plans (backward of combine)."""
        res = self.ll_dispatch(xs, [p.topk_idx for p in plans], [p.topk_w for p in plans], plans[0].num_experts, mode,
                               cpu_sync=False, stream=stream)
        return [(rx[:p.num_rows], None if rsf is None else rsf[:p.num_rows]) for (_, rx, rsf), p in zip(res, plans)]

    def ll_combine(self, xs: Sequence[torch.Tensor], plans: Sequence[RoutingPlan], stream=None, outs: Optional[list] = None):
        lay, dev = self.layout, self.device
        results, args = [], []
        for i, plan in enumerate(plans):
            out = outs[i] if outs is not None else torch.empty((plan.num_tokens, lay.hidden), dtype=torch.bfloat16, device=dev)
            results.append(out)
            args.append(dict(x=xs[i].data_ptr(), recv_row_src=plan.recv_row_src.data_ptr(), num_rows=plan.num_rows_dev.data_ptr(),
                             topk_idx=plan.topk_idx.data_ptr(), topk_w=plan.topk_w.data_ptr(), T=plan.num_tokens,
                             E=plan.num_experts, out=out.data_ptr()))
        self._timed("ll_combine", stream, lambda: self.C.ll_combine(lay, self.sessions, args, self.ll_blocks(), self._stream(stream),
                                                                           self._device_profile))
        return results

    def barrier(self, stream=None) -> None:
        self.C.barrier(self.sessions, self._stream(stream))
