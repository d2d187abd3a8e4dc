"""The upstream V1 workflow (layout -> dispatch -> combine, cached dispatch, six-tensor handle) on two Gloo ranks,
against the all-rank oracle."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deepep_b200.oracle import reference as R
from helpers import bits_equal, make_routes, make_weights

WORLD, H, E, K = 2, 128, 8, 3
TOKENS = [50, 23]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD, timeout=__import__("datetime").timedelta(seconds=120))
    import deepep_b200 as deep_ep

    xs = [torch.randn((t, H), generator=torch.Generator().manual_seed(r)).bfloat16() for r, t in enumerate(TOKENS)]
    idx = [make_routes("invalid", t, E, K, WORLD, 3 + r) for r, t in enumerate(TOKENS)]
    ws = [make_weights(t, K, r) for r, t in enumerate(TOKENS)]
    ref, lays = R.dispatch(xs, idx, ws, E, do_expand=False)
    local = E // WORLD
    buf = deep_ep.Buffer(dist.group.WORLD, num_max_tokens_per_rank=64, hidden=H, num_topk=K)
    checks = {}
    per_rank, per_rdma, per_expert, in_rank, _ = buf.get_dispatch_layout(idx[rank], E)
    dest = torch.where(idx[rank] >= 0, idx[rank] // local, torch.full_like(idx[rank], -1))
    want_in_rank = torch.stack([(dest == d).any(1) for d in range(WORLD)], 1)
    checks["layout"] = (per_rdma is None and torch.equal(in_rank, want_in_rank) and per_rank.tolist() == want_in_rank.sum(0).tolist()
                        and per_expert.tolist() == torch.bincount(idx[rank][idx[rank] >= 0], minlength=E).tolist())
    rx, ridx, rw, counts, handle, _ = buf.dispatch(xs[rank], topk_idx=idx[rank], topk_weights=ws[rank], num_tokens_per_rank=per_rank,
                                                   is_token_in_rank=in_rank, num_tokens_per_expert=per_expert)
    checks["dispatch"] = bits_equal(rx, ref[rank][0]) and torch.equal(ridx, ref[rank][1]) and torch.equal(rw, ref[rank][2])
    checks["counts"] = list(counts) == [int((ridx == l).sum()) for l in range(local)]
    rank_prefix, chan_prefix, recv_chan_prefix, recv_src_idx, in_rank2, send_head = handle
    # rank_prefix[i][j]: rows that rank j receives from ranks 0..i
    want_prefix = torch.tensor([[int(lays[j].rank_rows[:i + 1].sum()) for j in range(WORLD)] for i in range(WORLD)])
    checks["handle"] = (torch.equal(rank_prefix.long(), want_prefix) and torch.equal(in_rank2, in_rank)
                        and torch.equal(recv_src_idx.long(), lays[rank].row_token.long())
                        and torch.equal(send_head[:, rank] >= 0, in_rank[:, rank]))
    out, ow, _ = buf.combine(rx, handle, topk_weights=rw)
    cref = R.combine([r_[0] for r_ in ref], lays, TOKENS, K, topk_weights=[r_[2] for r_ in ref])
    checks["combine"] = bits_equal(out, cref[rank][0]) and torch.equal(ow, cref[rank][1])
    again = buf.dispatch(xs[rank], handle=handle)[0]                      # cached dispatch: same rows without a layout pass
    checks["cached"] = bits_equal(again, ref[rank][0])
    buf.destroy()
    # a buffer sized on first use: the ranks' batches differ (50 and 23 tokens), the workspace they agree on does not
    lazy = deep_ep.Buffer(dist.group.WORLD)
    rx2 = lazy.dispatch(xs[rank], topk_idx=idx[rank], topk_weights=ws[rank], num_tokens_per_expert=per_expert)[0]
    checks["lazy"] = bits_equal(rx2, ref[rank][0]) and lazy._elastic.num_max_tokens_per_rank == max(TOKENS)
    lazy.destroy()
    results[rank] = checks
    dist.destroy_process_group()


def test_v1_workflow_on_gloo_ranks():
    port = _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(port, results), nprocs=WORLD, join=True)
        for rank in range(WORLD):
            assert all(results[rank].values()), (rank, results[rank])
