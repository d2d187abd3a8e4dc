"""The fused MoE forward (MXFP8 activations, MXFP4 weights, one shared expert per rank) through the public API.

    python examples/mega_moe.py
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/mega_moe.py
The ranks meet through the launcher's TCPStore (a ``StoreGroup``; no process group is needed).  On GPUs this is one
persistent tcgen05 kernel per rank; without a GPU the same calls run on the CPU engine (small shapes only).
Parity: ``example.py`` of the reference's megamoe package.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from deep_ep_experimental.megamoe import StoreGroup, SymmBuffer, fp8_fp4_mega_moe, transform_weights_for_mega_moe  # noqa: E402
from deepep_b200.oracle import megamoe as O  # noqa: E402
from deepep_b200.utils.math import per_token_cast_to_fp8  # noqa: E402


def main():
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    hidden, intermediate, topk, local_experts = (2048, 1024, 4, 8) if cuda else (256, 128, 2, 2)
    num_experts, tokens = local_experts * world, 64 if cuda else 6
    group = StoreGroup.from_env() if world > 1 else None
    try:
        buffer = SymmBuffer(group, num_experts=num_experts, num_max_tokens_per_rank=tokens, num_topk=topk, hidden=hidden,
                            intermediate_hidden=intermediate, num_shared_experts=1)
        # this rank's routed experts and its shared expert: packed e2m1 pairs + ue8m0 scales per 32 values
        l1, l2 = O.make_weights(local_experts, hidden, intermediate, seed=100 + rank)
        s1, s2 = O.make_weights(1, hidden, intermediate, seed=900 + rank)
        w1, w2 = transform_weights_for_mega_moe(l1, l2, device=device)                  # once per weight set
        shared_w1, shared_w2 = transform_weights_for_mega_moe(s1, s2, shared=True, device=device)

        g = torch.Generator().manual_seed(rank)
        x = torch.randn((tokens, hidden), generator=g).bfloat16().to(device)
        topk_idx = torch.rand((tokens, num_experts), generator=g).topk(topk, dim=1).indices.to(device)
        topk_weights = torch.softmax(torch.randn((tokens, topk), generator=g), dim=1).to(device)
        x_fp8, x_sf = per_token_cast_to_fp8(x, use_ue8m0=True)                          # e4m3 + power-of-two scales per 128
        buffer.load_inputs(x_fp8, x_sf, topk_idx, topk_weights)
        buffer.validate_inputs(tokens)

        y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device)
        stats = torch.zeros(local_experts, dtype=torch.int32, device=device)
        fp8_fp4_mega_moe(y, w1, w2, buffer, shared_l1_weights=shared_w1, shared_l2_weights=shared_w2,
                         cumulative_local_expert_recv_stats=stats)
        if cuda:
            torch.cuda.synchronize()
        finite = bool(torch.isfinite(y.float()).all())
        print(f"rank {rank}/{world} on {device}: y {tuple(y.shape)}, |y| mean {y.float().abs().mean().item():.4f}, "
              f"rows per local expert {stats.tolist()}: {'ok' if finite else 'WRONG'}", flush=True)
        if group is not None:
            group.barrier("before teardown")
        buffer.destroy()
        if group is not None:
            group.close()
    except BaseException as error:
        if group is not None:
            group.abort(f"MegaMoE example: {type(error).__name__}: {error}")
        raise
    return 0 if finite else 1


if __name__ == "__main__":
    sys.exit(main())
