"""Expert-parallel dispatch -> experts -> combine, forward and backward, through the public API.

    python examples/dispatch_combine.py                                                        # one process
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/dispatch_combine.py
One process per GPU with NCCL as the control plane; without a GPU the same script runs on the CPU engine over Gloo.
The "experts" scale every row by its routing weight, so the result can be checked against ``sum_k w_k * x``.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import deep_ep  # noqa: E402


def main():
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    group = None
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": device} if cuda else {}))
        group = dist.group.WORLD
    tokens, hidden, num_experts, num_topk = 512, 1024, 8 * world, 4
    buffer = deep_ep.ElasticBuffer(group, num_max_tokens_per_rank=tokens, hidden=hidden, num_topk=num_topk,
                                   explicitly_destroy=True)
    g = torch.Generator().manual_seed(rank)
    x = torch.randn((tokens, hidden), generator=g).bfloat16().to(device)
    scores = torch.rand((tokens, num_experts), generator=g)
    topk_weights, topk_idx = torch.topk(torch.softmax(scores, dim=1), num_topk, dim=1)
    topk_idx, topk_weights = topk_idx.to(device), topk_weights.float().contiguous().to(device)

    # forward: rows arrive sorted by (local expert, source rank, source token, slot)
    recv_x, _, recv_w, handle, _ = buffer.dispatch(x, topk_idx=topk_idx, topk_weights=topk_weights, num_experts=num_experts,
                                                   do_expand=True)
    counts = handle.num_recv_tokens_per_expert_list                      # rows of every local expert, for a grouped matmul
    expert_out = (recv_x.float() * recv_w[:, None]).bfloat16()
    out, _, _ = buffer.combine(expert_out, handle)
    error = (out.float() - x.float() * topk_weights.sum(1, keepdim=True)).abs().max().item()

    # backward by handle reversal
    grad_out = torch.randn((tokens, hidden), generator=g).bfloat16().to(device)
    grad_expert_out = buffer.dispatch(grad_out, handle=handle)[0]                       # backward of combine
    grad_recv_x = (grad_expert_out.float() * recv_w[:, None]).bfloat16()
    grad_recv_w = (grad_expert_out.float() * recv_x.float()).sum(1)
    grad_x, grad_w, _ = buffer.combine(grad_recv_x, handle, topk_weights=grad_recv_w)  # backward of dispatch
    grad_error = (grad_x.float() - grad_out.float() * topk_weights.sum(1, keepdim=True)).abs().max().item()

    ok = error < 0.1 and grad_error < 0.2 and tuple(grad_w.shape) == (tokens, num_topk) and sum(counts) == recv_x.shape[0]
    print(f"rank {rank}/{world} on {device}: received {recv_x.shape[0]} rows for {len(counts)} local experts, "
          f"max error {error:.4f} (forward) {grad_error:.4f} (backward): {'ok' if ok else 'WRONG'}", flush=True)
    buffer.destroy()
    if world > 1:
        dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
