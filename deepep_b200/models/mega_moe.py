"""MegaMoE: the fused expert-parallel MoE forward (fp8 activations x fp4 weights).

Public API (parity: ``experiments/megamoe/python/deep_ep_experimental/megamoe/api.py`` of the reference:
``SymmBuffer`` :63-282, ``transform_weights_for_mega_moe`` :311-379, ``fp8_fp4_mega_moe`` :382-517,
``mega_moe`` :520-567):

    buf = SymmBuffer(group, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden)
    l1, l2 = transform_weights_for_mega_moe((w1, w1_sf), (w2, w2_sf))
    buf.x[:bs] = ...; buf.x_sf[:bs] = ...; buf.topk_idx[:bs] = ...; buf.topk_weights[:bs] = ...
    fp8_fp4_mega_moe(y, l1, l2, buf)          # y[:bs] is overwritten

Data path on each rank: (1) ``mega_route``: handshake, read every rank's routing table from peer memory,
lay local experts out as 128-row tiles, pull the routed e4m3 rows + ue8m0 scales over NVLink; (2) grouped
GEMM1 on tcgen05 with a SwiGLU + MXFP8 requantising epilogue; (3) grouped GEMM2 whose epilogue writes bf16
rows straight into the source rank's combine slots over NVLink; (4) ``mega_finish``: handshake, then
``y[t] = sum_k w[t, k] * row[t, k]`` in fp32.  The route weight is applied after the second GEMM.
"""
from __future__ import annotations

from dataclasses import dataclass
import os
from typing import Optional, Sequence, Tuple

import torch

from ..ops import require_native


class _DevicePointer:
    """Minimal ``__cuda_array_interface__`` holder so torch can view workspace memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _view(ptr: int, nbytes: int, device) -> torch.Tensor:
    return torch.as_tensor(_DevicePointer(ptr, nbytes), device=device)


@dataclass
class MegaWeights:
    """One projection of all local experts in kernel layout."""
    packed: torch.Tensor        # tiled uint8 [(L * N / 128) * (K / 128) * 128, 64 | 128]: e2m1 pairs (low nibble first) or e4m3
    sf_chunks: torch.Tensor     # 512-byte scale chunks
    experts: int
    n: int
    k: int
    fp8: bool = False           # e4m3 weights (mma_type "fp8xfp8") instead of e2m1 ("fp8xfp4")
    source: Optional[Tuple[torch.Tensor, torch.Tensor]] = None   # (weights, scales) as given; kept for CPU targets only


def _sf_chunks(sf: torch.Tensor) -> torch.Tensor:
    from ..oracle.megamoe import to_sf_chunks

    return to_sf_chunks(sf)


def transform_weights_for_mega_moe(l1_weights: Tuple[torch.Tensor, torch.Tensor], l2_weights: Tuple[torch.Tensor, torch.Tensor],
                                   activation: str = "swiglu", *, shared: bool = False, device=None) -> Tuple[MegaWeights, MegaWeights]:
    """Rearrange ``(w1 [L, 2I, H/2], w1_sf [L, 2I, H/32])`` and ``(w2 [L, H, I/2], w2_sf [L, H, I/32])`` for the kernel.

    Weights are packed e2m1 pairs (uint8, two values per byte: ``mma_type="fp8xfp4"``) or, for ``mma_type="fp8xfp8"``,
    e4m3 tensors ``w1 [L, 2I, H]`` / ``w2 [L, H, I]``; the scales are ue8m0 per 32 values either way.
    W1 rows are regrouped so every 256-row tile holds 128 gate rows followed by the 128 matching up rows
    (gate = first I rows, up = last I rows); scales go into the tensor-memory chunk layout.
    """
    if activation != "swiglu":
        raise NotImplementedError("only SwiGLU is implemented")
    del shared       # the reference lays shared experts out differently; here they use the routed experts' layout
    (w1, w1_sf), (w2, w2_sf) = l1_weights, l2_weights
    fp8 = w1.dtype == torch.float8_e4m3fn
    if (w2.dtype == torch.float8_e4m3fn) != fp8:
        raise ValueError("both projections must hold the same kind of weights")
    per_byte = 1 if fp8 else 2
    L, n1, hk = w1.shape
    inter, hidden = n1 // 2, hk * per_byte
    assert w2.shape == (L, hidden, inter // per_byte), "w2 must be [L, H, I / 2] (e2m1 pairs) or [L, H, I] (e4m3)"
    assert hidden % 256 == 0 and inter % 128 == 0, "hidden must be a multiple of 256, the intermediate size of 128"
    device = device or w1.device
    order = torch.arange(n1).view(2, inter // 128, 128).permute(1, 0, 2).reshape(-1)   # tile j: gate[128j:128j+128], up[128j:128j+128]
    from ..oracle.megamoe import tile_rows

    width = 128 // per_byte       # bytes of 128 K-values
    w1t = tile_rows(w1.view(torch.uint8)[:, order].reshape(L * n1, hk).contiguous(), width)
    w1_sft = w1_sf.view(torch.uint8).reshape(L, n1, hidden // 32)[:, order].reshape(L * n1, hidden // 32)
    w2t = tile_rows(w2.view(torch.uint8).reshape(L * hidden, inter // per_byte).contiguous(), width)
    w2_sft = w2_sf.view(torch.uint8).reshape(L * hidden, inter // 32)
    on_cpu = torch.device(device).type == "cpu"      # the CPU engine evaluates the restatement from the weights as given
    return (MegaWeights(w1t.to(device), _sf_chunks(w1_sft).to(device), L, n1, hidden, fp8, (w1, w1_sf) if on_cpu else None),
            MegaWeights(w2t.to(device), _sf_chunks(w2_sft).to(device), L, hidden, inter, fp8, (w2, w2_sf) if on_cpu else None))


class MegaEngine:
    """Runs the four kernels for one rank, or for several virtual ranks that share a GPU."""

    def __init__(self, sessions: Sequence, layout, device, num_experts: int, intermediate: int, num_sms: int = 0,
                 num_shared_experts: int = 0):
        self.C = require_native("MegaMoE")
        self.sessions, self.layout, self.device = list(sessions), layout, device
        self.n, self.world = len(self.sessions), layout.world
        self.M, self.H, self.K = layout.max_tokens, layout.hidden, layout.topk
        self.E, self.I = num_experts, intermediate
        self.L = num_experts // self.world
        self.S = int(num_shared_experts)              # shared experts: extra local experts that take all of this rank's tokens
        assert self.H % 256 == 0 and self.I % 128 == 0 and num_experts % self.world == 0
        assert self.S >= 0 and self.K + self.S <= 16, "top-k plus shared experts must not exceed 16"
        off = self.C.mega_input_offsets(self.M, self.H, self.K)
        self.in_off = layout.mega
        self.off_hdr, self.off_x, self.off_sf, self.off_idx, self.off_w, in_total = off
        self.comb_off = layout.mega + in_total        # combine slots [M][K + S][H] bf16
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self.gemm_blocks = num_sms or self.sm_count
        # tiles handed out by an atomic counter (default) or statically round-robin (DEEPEP_MEGA_STATIC_TILES=1)
        self.dynamic_tiles = os.environ.get("DEEPEP_MEGA_STATIC_TILES", "0") in ("", "0")
        # GEMM2 tiles scheduled after all GEMM1 tiles (0, the default) or right after their GEMM1 wave, which spreads the
        # combine rows over the kernel instead of its last third.  The value is the wave length in units of two rounds of
        # GEMM1 tiles over the CTAs (DEEPEP_MEGA_INTERLEAVE=<units>); off was the faster setting at 1, 2 and 4 GPUs.
        default = "0"
        self.interleave = int(os.environ.get("DEEPEP_MEGA_INTERLEAVE", default) or 0)   # wave length in units of two CTA rounds
        # CTA pairs (clusters of two CTAs share every weights tile: tcgen05.mma.cta_group::2): off by default, the fused
        # layer is as fast without them and experts padded to whole pairs of 128-row tiles carry more rows.
        # DEEPEP_MEGA_PAIRS=1 turns them on, "auto" uses them when the local experts average 384 rows or more.
        # Only with one rank per GPU: virtual ranks share the SMs.
        self.pairs = os.environ.get("DEEPEP_MEGA_PAIRS", "0").lower()
        if self.pairs not in ("auto", "0", "1"):
            raise ValueError("DEEPEP_MEGA_PAIRS must be auto, 0 or 1")
        rows = self.world * self.M * min(self.K, self.L) + self.S * self.M + (self.L + self.S) * 255   # room for whole pairs
        self.max_mtiles = -(-rows // 256) * 2
        self.rows_cap = self.max_mtiles * 128
        u8, i32 = dict(dtype=torch.uint8, device=device), dict(dtype=torch.int32, device=device)
        self.scratch = []
        for _ in range(self.n):
            self.scratch.append(dict(
                a1=torch.empty((self.rows_cap, self.H), **u8), a1_sf=torch.zeros((self.max_mtiles * (self.H // 128) * 512,), **u8),
                a2=torch.empty((self.rows_cap, self.I), **u8), a2_sf=torch.zeros((self.max_mtiles * (self.I // 128) * 512,), **u8),
                row_src=torch.empty((self.rows_cap,), **i32), mtile_expert=torch.zeros((self.max_mtiles,), **i32),
                num_mtiles=torch.zeros((1,), **i32), expert_rows=torch.zeros((self.L + self.S,), **i32),
                expert_list=torch.empty(((self.L + self.S) * self.world * self.M,), **i32), err=torch.zeros((1,), **i32),
                ready=torch.zeros((self.max_mtiles,), **i32), pulled=torch.zeros((self.max_mtiles,), **i32), tile_counter=torch.zeros((1,), **i32)))

    @staticmethod
    def mega_bytes(C, max_tokens: int, hidden: int, topk: int, num_shared_experts: int = 0) -> int:
        return C.mega_input_offsets(max_tokens, hidden, topk)[5] + max_tokens * (topk + num_shared_experts) * hidden * 2 + 1024

    def input_views(self, i: int):
        """(x e4m3 [M, H], x_sf uint8 [M, H/32], topk_idx int32 [M, K], topk_weights fp32 [M, K]) of rank slot i."""
        base = self.sessions[i].workspace + self.in_off
        M, H, K = self.M, self.H, self.K
        x = _view(base + self.off_x, M * H, self.device).view(torch.float8_e4m3fn).view(M, H)
        sf = _view(base + self.off_sf, M * (H // 32), self.device).view(M, H // 32)
        idx = _view(base + self.off_idx, M * K * 4, self.device).view(torch.int32).view(M, K)
        w = _view(base + self.off_w, M * K * 4, self.device).view(torch.float32).view(M, K)
        return x, sf, idx, w

    def forward(self, ys: Sequence[torch.Tensor], tokens: Sequence[int], l1: Sequence[MegaWeights], l2: Sequence[MegaWeights],
                stream=None, fused: bool = True, x_bf16: Optional[Sequence[Optional[torch.Tensor]]] = None,
                timer: Optional[torch.Tensor] = None) -> None:
        """Run the layer.  ``fused``: one persistent cooperative kernel (route -> GEMM1 -> GEMM2 -> finish); otherwise
        the same phases as four launches (kept for debugging and for comparing the two schedules).
        ``l1`` / ``l2`` hold the routed experts followed by the shared ones when the engine has shared experts.
        ``x_bf16[i]``: bf16 activations quantised to MXFP8 inside the kernel instead of pre-quantised inputs.
        ``timer``: int64 ``[SMs, mega_timer_words]`` that receives one record of phase stamps per CTA (fused, one rank)."""
        C, lay = self.C, self.layout
        s = (stream if stream is not None else torch.cuda.current_stream(self.device)).cuda_stream
        route_args, finish_args, gemm1_args, gemm2_args = [], [], [], []
        for i in range(self.n):
            sc, w1, w2 = self.scratch[i], l1[i], l2[i]
            route_args.append(dict(in_off=self.in_off, T=tokens[i], E=self.E, K=self.K, H=self.H, max_tokens=self.M,
                                   S=self.S, x_bf16=None if x_bf16 is None or x_bf16[i] is None else x_bf16[i].data_ptr(),
                                   timer=None if timer is None else timer.data_ptr(),
                                   max_mtiles=self.max_mtiles, a1=sc["a1"].data_ptr(), a1_sf=sc["a1_sf"].data_ptr(),
                                   row_src=sc["row_src"].data_ptr(), mtile_expert=sc["mtile_expert"].data_ptr(),
                                   num_mtiles=sc["num_mtiles"].data_ptr(), expert_rows=sc["expert_rows"].data_ptr(),
                                   expert_list=sc["expert_list"].data_ptr()))
            finish_args.append(dict(in_off=self.in_off, comb_off=self.comb_off, T=tokens[i], E=self.E, K=self.K, H=self.H,
                                    max_tokens=self.M, y=ys[i].data_ptr(), S=self.S,
                                    timer=None if timer is None else timer.data_ptr()))
            common = dict(mtile_expert=sc["mtile_expert"].data_ptr(), num_mtiles=sc["num_mtiles"].data_ptr(), rows_pad=self.rows_cap,
                          error_flag=sc["err"].data_ptr())
            gemm1_args.append(dict(common, a=sc["a1"].data_ptr(), sfa=sc["a1_sf"].data_ptr(), b=w1.packed.data_ptr(),
                                   sfb=w1.sf_chunks.data_ptr(), k=self.H, b_rows=w1.experts * w1.n, n_total=w1.n, epi=1,
                                   b_fp8=int(w1.fp8),
                                   a2=sc["a2"].data_ptr(), a2_sf=sc["a2_sf"].data_ptr(), inter=self.I))
            gemm2_args.append(dict(common, a=sc["a2"].data_ptr(), sfa=sc["a2_sf"].data_ptr(), b=w2.packed.data_ptr(),
                                   sfb=w2.sf_chunks.data_ptr(), k=self.I, b_rows=w2.experts * w2.n, n_total=w2.n, epi=2,
                                   b_fp8=int(w2.fp8),
                                   row_src=sc["row_src"].data_ptr(), comb_off=self.comb_off, max_tokens=self.M,
                                   topk=self.K + self.S, hidden=self.H))
        if fused:
            pair = self.use_pairs(tokens)
            for i in range(self.n):    # the fused kernel overlaps the pull with the GEMMs through per-tile counters
                sc = self.scratch[i]
                route_args[i]["pulled"] = sc["pulled"].data_ptr()
                route_args[i]["tile_pairs"] = int(pair)
                gemm1_args[i]["a_ready"] = sc["pulled"].data_ptr()
            blocks = max(1, min(self.gemm_blocks, self.sm_count // self.n))
            C.mega_fused(lay, self.sessions, [dict(route=route_args[i], finish=finish_args[i], gemm1=gemm1_args[i],
                                                  gemm2=gemm2_args[i], ready=self.scratch[i]["ready"].data_ptr(),
                                                  tile_counter=self.scratch[i]["tile_counter"].data_ptr() if self.dynamic_tiles else None,
                                                  interleave=int(self.interleave), pair=int(pair))
                                             for i in range(self.n)], blocks, s)
            return
        aux_blocks = max(1, min(self.sm_count // self.n, 128))
        C.mega_route(lay, self.sessions, route_args, aux_blocks, s)
        for i in range(self.n):
            C.mega_gemm(gemm1_args[i], self.sessions[i], self.gemm_blocks, s)
            C.mega_gemm(gemm2_args[i], self.sessions[i], self.gemm_blocks, s)
        C.mega_finish(lay, self.sessions, finish_args, aux_blocks, s)

    def use_pairs(self, tokens: Sequence[int]) -> bool:
        """Whether this launch runs its GEMMs as CTA pairs (see ``self.pairs``)."""
        if self.n != 1 or self.pairs == "0" or self.sm_count < 2:
            return False
        if self.pairs == "1":
            return True
        # expected rows per local expert if every rank sends what this one does, spread evenly over the experts
        per_expert = self.world * max(tokens) * self.K / max(self.E, 1) if self.L else 0
        return per_expert >= 384

    WAIT_SITES = {1: "a pipeline barrier", 2: "the tile ticket from the producer warp", 3: "the first projection of a row block",
                  4: "rows pulled from the peers", 5: "the release of a group of operand stages", 6: "the drain of an accumulator",
                  7: "the drain of the partner CTA's accumulator", 8: "operands arriving in a stage", 9: "a finished accumulator",
                  10: "the epilogue of the previous tile"}

    def check(self) -> None:
        """Raises when a wait inside the kernel ran out, naming what the CTA was waiting for (the kernel's ``GemmWaitSite``)."""
        for i, sc in enumerate(self.scratch):
            code = int(sc["err"].item())
            if code != 0:
                raise RuntimeError(f"a wait ran out inside the MegaMoE kernel of local rank {i}: it was waiting for "
                                   f"{self.WAIT_SITES.get(code, f'site {code}')}")


class MegaCpuEngine:
    """The fused MoE forward without a GPU: every rank gathers all ranks' expert weights and routing tables through the
    control plane and evaluates the CPU restatement (``oracle/megamoe.py``) for its own tokens.  Meant for tests of the
    API on Gloo or store-only ranks, with small shapes."""

    def __init__(self, control, num_experts: int, num_shared_experts: int):
        self.control, self.E, self.S = control, num_experts, int(num_shared_experts)
        self.L = num_experts // control.size
        self.sm_count = 0

    @staticmethod
    def _source(weights: MegaWeights, what: str):
        if weights.source is None:
            raise ValueError(f"{what} were transformed for a GPU; pass device='cpu' to transform_weights_for_mega_moe")
        return weights.source

    def forward(self, y: torch.Tensor, sym: "SymmBuffer", l1: MegaWeights, l2: MegaWeights, shared_l1: Optional[MegaWeights],
                shared_l2: Optional[MegaWeights], x_bf16: Optional[torch.Tensor], stats: Optional[torch.Tensor]) -> None:
        from ..oracle import megamoe as O

        bs = y.shape[0]
        codes, sf = O.quantize_mxfp8(x_bf16) if x_bf16 is not None else (sym.x[:bs], sym.x_sf[:bs])
        idx, w = sym.topk_idx[:bs].long(), sym.topk_weights[:bs]
        parts = self.control.all_gather_object((self._source(l1, "l1 weights"), self._source(l2, "l2 weights"), idx))
        cat = lambda which, item: torch.cat([p[which][item] for p in parts])
        everyone1, everyone2 = (cat(0, 0), cat(0, 1)), (cat(1, 0), cat(1, 1))
        own1 = None if shared_l1 is None else self._source(shared_l1, "shared l1 weights")
        own2 = None if shared_l2 is None else self._source(shared_l2, "shared l2 weights")
        y.copy_(O.mega_moe_reference([(codes, sf)], [idx], [w], everyone1, everyone2, self.E, own1, own2)[0])
        if stats is not None:       # rows every routed local expert received from all ranks (first occurrence of an id in a row)
            mine = torch.zeros(self.L, dtype=torch.int64)
            for p in parts:
                t = p[2]
                first = torch.ones_like(t, dtype=torch.bool)
                for k in range(1, t.shape[1]):
                    first[:, k] = ~(t[:, :k] == t[:, k:k + 1]).any(dim=1)
                hit = t[first & (t >= self.control.rank * self.L) & (t < (self.control.rank + 1) * self.L)] - self.control.rank * self.L
                mine += torch.bincount(hit, minlength=self.L)
            stats.add_(mine.to(stats.dtype))

    def check(self) -> None:
        return None


class SymmBuffer:
    """Symmetric input/output block of the fused MoE forward; construction is collective."""

    def __init__(self, group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int, hidden: int,
                 intermediate_hidden: int, num_shared_experts: int = 0, mma_type: str = "fp8xfp4", activation: str = "swiglu",
                 *, ranks_per_node: int = 0, timeout: Optional[float] = None, rank: Optional[int] = None,
                 world_size: Optional[int] = None, device=None, num_gpu_timeout_secs: float = 100, num_sms: int = 0):
        """``group``: a process group, a ``StoreGroup``, or ``None`` (one process, or ``rank=`` / ``world_size=`` over the
        launcher's TCPStore).  ``ranks_per_node`` is accepted for the reference's signature (``api.py:70-84``; all ranks
        share one NVLink domain here); ``timeout`` (seconds), when given, is the limit of the host-side waits of the
        set-up and of the waits inside the kernel (otherwise 300 s and ``num_gpu_timeout_secs``)."""
        del ranks_per_node
        if timeout is not None:
            num_gpu_timeout_secs = float(timeout)
        if mma_type not in ("fp8xfp4", "fp8xfp8"):
            raise ValueError("mma_type must be 'fp8xfp4' (e2m1 weights) or 'fp8xfp8' (e4m3 weights)")
        if activation != "swiglu":
            raise NotImplementedError("only SwiGLU is implemented")
        from ..parallel.runtime import ControlPlane, Runtime

        self.control = ControlPlane(group, rank, world_size, timeout=300.0 if timeout is None else float(timeout))
        self.rank, self.world_size = self.control.rank, self.control.size
        self.num_experts, self.num_topk, self.hidden, self.intermediate_hidden = num_experts, num_topk, hidden, intermediate_hidden
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.num_shared_experts, self.mma_type = int(num_shared_experts), mma_type
        self._joined: dict = {}
        self.batch_size = 0
        self._destroyed = False
        if not torch.cuda.is_available() or (device is not None and torch.device(device).type == "cpu"):
            # no GPU: plain tensors for the inputs and the CPU restatement as the engine (tests of the API on CPU ranks)
            if num_experts % self.world_size or hidden % 256 or intermediate_hidden % 128 or num_topk + self.num_shared_experts > 16:
                raise ValueError("experts must divide by the world size, hidden by 256, the intermediate size by 128; top-k plus "
                                 "shared experts must not exceed 16")
            self.device, self.runtime, self.layout = torch.device("cpu"), None, None
            self.engine = MegaCpuEngine(self.control, num_experts, self.num_shared_experts)
            m = num_max_tokens_per_rank
            self.x = torch.zeros((m, hidden), dtype=torch.float8_e4m3fn)
            self.x_sf = torch.zeros((m, hidden // 32), dtype=torch.uint8)
            self.topk_idx = torch.full((m, num_topk), -1, dtype=torch.int32)
            self.topk_weights = torch.zeros((m, num_topk), dtype=torch.float32)
            self.control.barrier()
            return
        C = require_native("MegaMoE SymmBuffer")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        mega = MegaEngine.mega_bytes(C, num_max_tokens_per_rank, hidden, num_topk, self.num_shared_experts)
        # the generic regions are sized for one token: this buffer only uses the fused-MoE region
        self.layout = C.make_mega_layout(self.world_size, num_max_tokens_per_rank, hidden, num_topk, mega)
        self.runtime = Runtime(self.control, self.layout, float(num_gpu_timeout_secs), self.device)
        self.engine = MegaEngine([self.runtime.native], self.layout, self.device, num_experts, intermediate_hidden, num_sms,
                                 self.num_shared_experts)
        # self._joined: routed + shared weights joined once per weight set
        self.x, self.x_sf, self.topk_idx, self.topk_weights = self.engine.input_views(0)

    def prepare(self, batch_size: int) -> "SymmBuffer":
        if not 0 <= batch_size <= self.num_max_tokens_per_rank:
            raise ValueError(f"batch size must be in [0, {self.num_max_tokens_per_rank}]")
        self.batch_size = batch_size
        return self

    def load_inputs(self, x: torch.Tensor, x_sf: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor) -> "SymmBuffer":
        """Copy one batch into the symmetric input block and ``prepare`` it.

        ``x`` is e4m3 ``[bs, hidden]``.  ``x_sf`` is either ue8m0 codes, uint8 ``[bs, hidden / 32]`` (the kernel's
        native form), or fp32 ``[bs, hidden / 128]`` block scales that are powers of two (what
        ``per_token_cast_to_fp8(x, use_ue8m0=True)`` produces): those are exact in ue8m0 and each is used for its four
        32-value blocks.  Other fp32 scales would have to be rounded, which changes the numbers, so they are refused.
        """
        bs = x.shape[0]
        if x.dtype != torch.float8_e4m3fn or tuple(x.shape) != (bs, self.hidden) or bs > self.num_max_tokens_per_rank:
            raise ValueError(f"x must be e4m3 [batch <= {self.num_max_tokens_per_rank}, {self.hidden}]")
        if x_sf.dtype == torch.uint8 and tuple(x_sf.shape) == (bs, self.hidden // 32):
            codes = x_sf
        elif x_sf.dtype == torch.float32 and tuple(x_sf.shape) == (bs, self.hidden // 128):
            mantissa, exponent = torch.frexp(x_sf)            # x_sf = mantissa * 2^exponent, mantissa in [0.5, 1)
            if not bool((mantissa == 0.5).all()) or not bool(((exponent >= -126) & (exponent <= 128)).all()):
                raise ValueError("fp32 block scales must be powers of two (per_token_cast_to_fp8(x, use_ue8m0=True)); "
                                 "other scales cannot be carried by the ue8m0 scale format without rounding")
            codes = (exponent - 1 + 127).to(torch.uint8).repeat_interleave(4, dim=1)
        else:
            raise ValueError("x_sf must be uint8 [batch, hidden / 32] (ue8m0) or fp32 [batch, hidden / 128] (powers of two)")
        self.x.view(torch.uint8)[:bs].copy_(x.view(torch.uint8))
        self.x_sf[:bs].copy_(codes)
        self.topk_idx[:bs].copy_(topk_idx.to(torch.int32))
        self.topk_weights[:bs].copy_(topk_weights.float())
        return self.prepare(bs)

    def allocate_timer(self) -> torch.Tensor:
        """A zeroed int64 ``[SMs, words]`` tensor for ``fp8_fp4_mega_moe(..., timer=...)``: the kernel writes one record
        of phase stamps per CTA; ``mega_tools.parse_timer`` turns it into a per-phase breakdown.
        Parity: ``SymmBuffer.allocate_timer`` (``api.py:226-233`` of the reference)."""
        if self.runtime is None:
            raise NotImplementedError("the phase timer is written by the CUDA kernel; there is none on the CPU engine")
        C = require_native("MegaMoE timer")
        return torch.zeros((self.engine.sm_count, C.mega_timer_words), dtype=torch.int64, device=self.device)

    def joined_weights(self, routed: MegaWeights, shared: Optional[MegaWeights]) -> MegaWeights:
        """Routed experts followed by the shared ones in one operand (the kernel sees them as extra local experts)."""
        if shared is None:
            return routed
        key = (routed.packed.data_ptr(), shared.packed.data_ptr())
        if key not in self._joined:
            if (shared.n, shared.k, shared.fp8) != (routed.n, routed.k, routed.fp8):
                raise ValueError("shared experts must have the shapes and the weight type of the routed experts")
            self._joined[key] = MegaWeights(torch.cat([routed.packed, shared.packed]), torch.cat([routed.sf_chunks, shared.sf_chunks]),
                                            routed.experts + shared.experts, routed.n, routed.k, routed.fp8)
        return self._joined[key]

    def validate_inputs(self, batch_size: int, *, x: Optional[torch.Tensor] = None) -> None:
        """Scan the inputs of the next call (synchronises; keep it outside timed regions).  ``x``: the bf16 override that
        will be passed to ``fp8_fp4_mega_moe(..., x=...)``, if any (parity: ``api.py:235`` of the reference)."""
        if not 0 < batch_size <= self.num_max_tokens_per_rank:
            raise ValueError(f"batch size must be in [1, {self.num_max_tokens_per_rank}]")
        if x is not None and (x.dtype != torch.bfloat16 or tuple(x.shape) != (batch_size, self.hidden) or not x.is_contiguous()
                              or not bool(torch.isfinite(x.float()).all())):
            raise ValueError("the x override must be finite contiguous bf16 [batch, hidden]")
        idx = self.topk_idx[:batch_size]
        if bool(((idx >= self.num_experts)).any()):
            raise ValueError("topk_idx holds expert ids outside [0, num_experts)")
        if not bool(torch.isfinite(self.topk_weights[:batch_size]).all()):
            raise ValueError("topk_weights must be finite")

    def destroy(self) -> None:
        if not self._destroyed:
            self._destroyed = True
            if self.runtime is not None:
                self.runtime.close()
            else:
                self.control.barrier()


def fp8_fp4_mega_moe(y: torch.Tensor, l1_weights: MegaWeights, l2_weights: MegaWeights, sym_buffer: SymmBuffer,
                     shared_l1_weights: Optional[MegaWeights] = None, shared_l2_weights: Optional[MegaWeights] = None,
                     cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None, recipe=(1, 1, 32),
                     activation: str = "swiglu", activation_clamp=None, fast_math: bool = True, *, x: Optional[torch.Tensor] = None,
                     timer: Optional[torch.Tensor] = None, fused: bool = True, check: bool = False) -> None:
    """Fused MoE forward; overwrites ``y`` (bf16 ``[bs, hidden]``, ``bs = y.shape[0]``) in place and returns ``None``.

    The positional parameters follow the reference (``api.py:520-535``).  Inputs are read from ``sym_buffer.x`` /
    ``x_sf`` / ``topk_idx`` / ``topk_weights`` unless ``x`` (bf16 ``[bs, hidden]``) is given, which the kernel quantises
    to MXFP8 itself.  ``shared_l1_weights`` / ``shared_l2_weights`` (both or neither; transformed like the routed
    weights) are the rank's shared experts: every token passes through them with weight one.
    ``cumulative_local_expert_recv_stats`` (int32 ``[experts per rank]``) is incremented by the rows every routed
    local expert received.  ``timer``: see ``SymmBuffer.allocate_timer``.  ``check=True`` synchronises and raises if a
    wait inside the kernel ran out.
    """
    if tuple(recipe) != (1, 1, 32):
        raise NotImplementedError("the tensor-core path consumes one ue8m0 scale per 32 values: recipe must be (1, 1, 32)")
    if activation != "swiglu" or activation_clamp is not None or fast_math is not True:
        raise NotImplementedError("only unclamped SwiGLU with the default math is implemented")
    if not isinstance(sym_buffer, SymmBuffer):
        raise TypeError("sym_buffer must be a SymmBuffer of this library")
    if not isinstance(l1_weights, MegaWeights) or not isinstance(l2_weights, MegaWeights):
        raise TypeError("pass the weights through transform_weights_for_mega_moe first")
    if (shared_l1_weights is None) != (shared_l2_weights is None):
        raise ValueError("supply both shared weight pairs, or neither")
    shared = 0 if shared_l1_weights is None else shared_l1_weights.experts
    if shared != sym_buffer.num_shared_experts:
        raise ValueError("the shared expert count does not match the buffer's num_shared_experts")
    if y.dtype != torch.bfloat16 or y.dim() != 2 or y.shape[1] != sym_buffer.hidden or not y.is_contiguous():
        raise ValueError("y must be a contiguous bf16 [batch, hidden] tensor")
    bs = y.shape[0]
    if not 0 < bs <= sym_buffer.num_max_tokens_per_rank:
        raise ValueError("the batch must be non-empty and fit the buffer")
    if x is not None and (x.dtype != torch.bfloat16 or tuple(x.shape) != (bs, sym_buffer.hidden) or not x.is_contiguous()):
        raise ValueError("the x override must be contiguous bf16 [batch, hidden]; omit x for buffered fp8 input")
    if l1_weights.fp8 != (sym_buffer.mma_type == "fp8xfp8") or l2_weights.fp8 != l1_weights.fp8:
        raise ValueError(f"the buffer was built for mma_type={sym_buffer.mma_type!r}; the weights are of the other kind")
    if l1_weights.k != sym_buffer.hidden or l1_weights.n != 2 * sym_buffer.intermediate_hidden:
        raise ValueError("l1 weights do not match the buffer's hidden / intermediate sizes")
    if l1_weights.experts * sym_buffer.world_size != sym_buffer.num_experts:
        raise ValueError("each rank must hold num_experts / world_size experts")
    stats = cumulative_local_expert_recv_stats
    local = sym_buffer.num_experts // sym_buffer.world_size
    if stats is not None and (stats.dtype != torch.int32 or tuple(stats.shape) != (local,) or stats.device != y.device
                              or not stats.is_contiguous()):
        raise ValueError("cumulative stats must be contiguous int32 [experts per rank] on the buffer's device")
    if timer is not None and (not fused or timer.dtype != torch.int64 or not timer.is_contiguous()):
        raise ValueError("timer must come from SymmBuffer.allocate_timer() and needs the fused kernel")
    engine = sym_buffer.engine
    if isinstance(engine, MegaCpuEngine):
        if timer is not None:
            raise ValueError("timer must come from SymmBuffer.allocate_timer() and needs the fused kernel")
        engine.forward(y, sym_buffer, l1_weights, l2_weights, shared_l1_weights, shared_l2_weights, x, stats)
        return None
    engine.forward([y], [bs], [sym_buffer.joined_weights(l1_weights, shared_l1_weights)],
                   [sym_buffer.joined_weights(l2_weights, shared_l2_weights)], fused=fused,
                   x_bf16=None if x is None else [x], timer=timer)
    if stats is not None:
        stats.add_(engine.scratch[0]["expert_rows"][:local])
    if check:
        torch.cuda.synchronize(sym_buffer.device)
        engine.check()
    return None


def mega_moe(x, topk_idx: torch.Tensor, topk_weights: torch.Tensor, l1_weights: MegaWeights,
             l2_weights: MegaWeights, sym_buffer: SymmBuffer, *, shared_l1_weights: Optional[MegaWeights] = None,
             shared_l2_weights: Optional[MegaWeights] = None, out: Optional[torch.Tensor] = None,
             timer: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Explicit-input convenience API (parity: ``mega_moe``, ``api.py:380-412``): ``x`` is bf16 ``[bs, hidden]`` (quantised
    to MXFP8 here) or an ``(e4m3, ue8m0)`` pair that is copied as is; fills the symmetric inputs and runs the fused forward.
    Returns ``(y, per_call_counts)`` as the reference does: the output and, int32 ``[experts per rank]``, the rows every
    routed local expert received in this call."""
    if isinstance(x, (tuple, list)):
        codes, sf = x
    else:
        codes, sf = quantize_mxfp8_cuda(x)
    bs = codes.shape[0]
    sym_buffer.x[:bs].copy_(codes)
    sym_buffer.x_sf[:bs].copy_(sf)
    sym_buffer.topk_idx[:bs].copy_(topk_idx.to(torch.int32))
    sym_buffer.topk_weights[:bs].copy_(topk_weights.float())
    y = torch.empty((bs, sym_buffer.hidden), dtype=torch.bfloat16, device=codes.device) if out is None else out
    counts = torch.zeros(sym_buffer.num_experts // sym_buffer.world_size, dtype=torch.int32, device=y.device)
    fp8_fp4_mega_moe(y, l1_weights, l2_weights, sym_buffer.prepare(bs), shared_l1_weights, shared_l2_weights, counts, timer=timer)
    return y, counts


def quantize_mxfp8_cuda(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """MXFP8 quantiser in torch ops (any device): e4m3 codes and ue8m0 exponents per 32 values."""
    from ..oracle.megamoe import quantize_mxfp8

    return quantize_mxfp8(x)


__all__ = ["MegaCpuEngine", "MegaEngine", "MegaWeights", "SymmBuffer", "fp8_fp4_mega_moe", "mega_moe", "transform_weights_for_mega_moe"]
