"""The fused MoE API on two CPU ranks (CPU engine: every rank evaluates the restatement for its own tokens from the
gathered expert weights): each rank holds its slice of the experts, results must equal the all-rank restatement
bit for bit; shared experts, receive statistics, the bf16 input override and the store-only bootstrap included.
Parity: the reference's CPU-side MegaMoE tests (``experiments/megamoe/tests``), which compare the API with its golden.
"""
import os
from datetime import timedelta

import pytest
import torch
import torch.multiprocessing as mp

from deepep_b200.models import mega_tools as MT
from deepep_b200.oracle import megamoe as O

WORLD, H, I, E, K, TOKENS = 2, 256, 128, 4, 2, [9, 5]


def _worker(rank, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(WORLD))
    from deep_ep_experimental.megamoe import SymmBuffer, fp8_fp4_mega_moe, mega_moe, transform_weights_for_mega_moe

    checks = {}
    try:
        spec = MT.contract(world=WORLD, tokens=TOKENS, hidden=H, intermediate=I, experts=E, topk=K, seed=4)
        xs, idx, ws, l1, l2 = MT.make_case(spec)
        idx[0][0, 1] = -1                                                   # a masked slot
        L = E // WORLD
        mine = slice(rank * L, (rank + 1) * L)
        w1, w2 = transform_weights_for_mega_moe((l1[0][mine], l1[1][mine]), (l2[0][mine], l2[1][mine]))
        # the ranks meet through the launcher's TCPStore only (no process group), as the reference's MegaMoE does
        sym = SymmBuffer(None, E, 16, K, H, I, rank=rank, world_size=WORLD, timeout=60)
        checks["cpu_engine"] = sym.device.type == "cpu" and sym.runtime is None and (sym.rank, sym.world_size) == (rank, WORLD)
        bs = TOKENS[rank]
        sym.load_inputs(xs[rank][0], xs[rank][1], idx[rank], ws[rank])
        y = torch.zeros((bs, H), dtype=torch.bfloat16)
        stats = torch.zeros(L, dtype=torch.int32)
        assert fp8_fp4_mega_moe(y, w1, w2, sym, cumulative_local_expert_recv_stats=stats) is None
        golden = O.mega_moe_reference(xs, idx, ws, l1, l2, E)
        checks["routed"] = torch.equal(y, golden[rank])
        everyone = torch.cat(idx)
        checks["stats"] = stats.tolist() == torch.bincount(everyone[everyone >= 0], minlength=E)[mine].tolist()
        fp8_fp4_mega_moe(y, w1, w2, sym, cumulative_local_expert_recv_stats=stats)
        checks["stats_accumulate"] = stats.tolist() == (2 * torch.bincount(everyone[everyone >= 0], minlength=E)[mine]).tolist()
        # bf16 input: quantised to MXFP8 by the call itself; the explicit-input form does the same
        xb = O.dequantize_mxfp8(*xs[rank]).bfloat16()
        y2 = torch.zeros_like(y)
        fp8_fp4_mega_moe(y2, w1, w2, sym, x=xb)
        requant = [O.quantize_mxfp8(O.dequantize_mxfp8(*x).bfloat16()) for x in xs]
        want = O.mega_moe_reference(requant, idx, ws, l1, l2, E)[rank]
        y3, per_call = mega_moe(xb, idx[rank], ws[rank], w1, w2, sym)
        checks["bf16_input"] = (torch.equal(y2, want) and torch.equal(y3, want)
                                and per_call.tolist() == torch.bincount(everyone[everyone >= 0], minlength=E)[mine].tolist())
        with pytest.raises(NotImplementedError, match="timer"):
            sym.allocate_timer()
        sym.destroy()
        # one shared expert per rank (each rank its own weights): every local token passes through it with weight one
        s1, s2 = O.make_weights(1, H, I, 50 + rank)
        sw1, sw2 = transform_weights_for_mega_moe(s1, s2)
        sym = SymmBuffer(None, E, 16, K, H, I, num_shared_experts=1, rank=rank, world_size=WORLD, timeout=60)
        sym.load_inputs(xs[rank][0], xs[rank][1], idx[rank], ws[rank])
        fp8_fp4_mega_moe(y, w1, w2, sym, sw1, sw2)
        alone = O.mega_moe_reference([xs[rank]], [idx[rank]], [ws[rank]], l1, l2, E, s1, s2)[0]
        checks["shared"] = torch.equal(y, alone) and not torch.equal(y, golden[rank])
        with pytest.raises(ValueError, match="num_shared_experts"):
            fp8_fp4_mega_moe(y, w1, w2, sym)
        sym.destroy()
    except Exception as exc:          # surfaced by the parent
        import traceback

        checks["error"] = traceback.format_exc()
    results[rank] = checks


def test_fused_moe_api_on_two_cpu_ranks():
    from torch.distributed import TCPStore

    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    server = TCPStore("127.0.0.1", 0, None, True, timedelta(seconds=60), wait_for_workers=False)
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(server.port, results), nprocs=WORLD, join=True)
        got = dict(results)
    want = dict(cpu_engine=True, routed=True, stats=True, stats_accumulate=True, bf16_input=True, shared=True)
    for rank in range(WORLD):
        assert got[rank] == want, got[rank]


def test_weights_transformed_for_a_gpu_are_refused_by_the_cpu_engine():
    from deepep_b200.models import mega_moe as MM

    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    l1, l2 = O.make_weights(E, H, I, 0)
    w1, w2 = MM.transform_weights_for_mega_moe(l1, l2)
    assert w1.source is not None and torch.equal(w1.source[0], l1[0])
    w1.source = None                                     # what a transform for a GPU leaves
    sym = MM.SymmBuffer(None, E, 8, K, H, I)
    y = torch.zeros((3, H), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="device='cpu'"):
        MM.fp8_fp4_mega_moe(y, w1, w2, sym.prepare(3))
    with pytest.raises(ValueError):
        MM.SymmBuffer(None, E, 8, K, 200, I)
    sym.destroy()


def _readme_worker(rank, port, results):
    """The MegaMoE example of the reference's README (``README.md:232-272``) with the device lines taken out."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(WORLD),
                      LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(WORLD))
    from deep_ep_experimental.megamoe import StoreGroup, SymmBuffer, fp8_fp4_mega_moe, transform_weights_for_mega_moe

    spec = MT.contract(world=WORLD, tokens=[6, 6], hidden=H, intermediate=I, experts=E, topk=K, seed=8)
    xs, idx, ws, all_l1, all_l2 = MT.make_case(spec)
    mine = slice(rank * (E // WORLD), (rank + 1) * (E // WORLD))
    l1_weights, l2_weights = (all_l1[0][mine], all_l1[1][mine]), (all_l2[0][mine], all_l2[1][mine])
    shared_l1_weights, shared_l2_weights = O.make_weights(1, H, I, 70 + rank)
    x_fp8, x_sf, topk_idx, topk_weights = xs[rank][0], xs[rank][1], idx[rank].to(torch.int32), ws[rank]
    ok = False
    group = StoreGroup.from_env(timeout=60)
    try:
        buffer = SymmBuffer(
            group, num_experts=E, num_max_tokens_per_rank=16,
            num_topk=K, hidden=H, intermediate_hidden=I,
            num_shared_experts=1, mma_type="fp8xfp4",
            ranks_per_node=int(os.environ["LOCAL_WORLD_SIZE"]),
        )
        w1, w2 = transform_weights_for_mega_moe(l1_weights, l2_weights)
        shared_w1, shared_w2 = transform_weights_for_mega_moe(
            shared_l1_weights, shared_l2_weights, shared=True,
        )
        num_tokens = x_fp8.shape[0]
        buffer.x[:num_tokens].copy_(x_fp8)
        buffer.x_sf[:num_tokens].copy_(x_sf)
        buffer.topk_idx[:num_tokens].copy_(topk_idx)
        buffer.topk_weights[:num_tokens].copy_(topk_weights)
        buffer.validate_inputs(num_tokens)
        buffer.prepare(num_tokens)
        y = torch.empty((num_tokens, H), dtype=torch.bfloat16)
        fp8_fp4_mega_moe(
            y, w1, w2, buffer,
            shared_l1_weights=shared_w1, shared_l2_weights=shared_w2,
        )
        want = O.mega_moe_reference([xs[rank]], [idx[rank]], [ws[rank]], all_l1, all_l2, E, shared_l1_weights, shared_l2_weights)[0]
        ok = torch.equal(y, want)
        group.barrier("before SHMEM teardown")
        buffer.destroy()
        group.close()
    except BaseException as error:
        group.abort(f"MegaMoE: {type(error).__name__}: {error}")
        results[rank] = repr(error)
        raise
    results[rank] = ok


def test_the_fused_moe_example_of_the_reference_readme():
    from torch.distributed import TCPStore

    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    server = TCPStore("127.0.0.1", 0, None, True, timedelta(seconds=60), wait_for_workers=False)
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_readme_worker, args=(server.port, results), nprocs=WORLD, join=True)
        assert dict(results) == {0: True, 1: True}
