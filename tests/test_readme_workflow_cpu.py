"""The usage pattern of the reference's README (``README.md:146-219``), as a user would paste it: four helper functions
around ``dispatch`` / ``combine`` that always wait on the returned event (also for synchronous calls), forward and
backward of a layer whose experts multiply by the routing weight, against plain autograd.  One process, CPU engine."""
import pytest
import torch

import deep_ep
from helpers import make_routes, make_weights


def test_the_four_helper_functions_of_the_readme():
    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    max_tokens_per_rank, hidden, num_topk, num_experts = 64, 128, 4, 8
    buffer = deep_ep.ElasticBuffer(group=None, num_bytes=(8 << 30) if max_tokens_per_rank <= 256 else None,
                                   num_max_tokens_per_rank=max_tokens_per_rank, hidden=hidden, num_topk=num_topk,
                                   explicitly_destroy=True, device="cpu")

    def dispatch_forward(x, topk_idx, topk_weights):
        recv_x, _, recv_weights, handle, event = buffer.dispatch(
            x.detach().contiguous(), topk_idx=topk_idx.contiguous(), topk_weights=topk_weights.detach().contiguous(),
            num_experts=num_experts, do_expand=True)
        event.current_stream_wait()
        return recv_x, recv_weights, handle

    def dispatch_backward(grad_recv_x, grad_recv_weights, handle):
        grad_x, grad_weights, event = buffer.combine(grad_recv_x.detach().contiguous(), handle,
                                                     topk_weights=grad_recv_weights.detach().contiguous())
        event.current_stream_wait()
        return grad_x, grad_weights

    def combine_forward(expert_out, handle):
        out, _, event = buffer.combine(expert_out.detach().contiguous(), handle)
        event.current_stream_wait()
        return out

    def combine_backward(grad_out, handle):
        grad_expert_out, _, _, _, event = buffer.dispatch(grad_out.detach().contiguous(), handle=handle)
        event.current_stream_wait()
        return grad_expert_out

    tokens = 50
    x = torch.randint(-3, 4, (tokens, hidden)).to(torch.bfloat16)          # small integers: sums are exact in bf16
    topk_idx = make_routes("invalid", tokens, num_experts, num_topk, 1, 3)
    topk_weights = torch.randint(1, 4, (tokens, num_topk)).float()
    # forward: experts scale every row by its routing weight
    recv_x, recv_weights, handle = dispatch_forward(x, topk_idx, topk_weights)
    expert_out = (recv_x.float() * recv_weights[:, None]).bfloat16()
    out = combine_forward(expert_out, handle)
    valid = (topk_idx >= 0).float()
    assert torch.equal(out.float(), x.float() * (topk_weights * valid).sum(1, keepdim=True))
    # backward of out = sum_k w_k x through the same handle
    grad_out = torch.randint(-2, 3, (tokens, hidden)).to(torch.bfloat16)
    grad_expert_out = combine_backward(grad_out, handle)
    grad_recv_x = (grad_expert_out.float() * recv_weights[:, None]).bfloat16()
    grad_recv_weights = (grad_expert_out.float() * recv_x.float()).sum(1)
    grad_x, grad_topk_weights = dispatch_backward(grad_recv_x, grad_recv_weights, handle)
    xr, wr = x.float().requires_grad_(), topk_weights.clone().requires_grad_()
    (xr * (wr * valid).sum(1, keepdim=True)).backward(grad_out.float())
    assert torch.equal(grad_x.float(), xr.grad) and torch.equal(grad_topk_weights, wr.grad)
    buffer.destroy()
    buffer.destroy()                                                        # idempotent


def test_waiting_on_an_empty_overlap_is_harmless():
    ev = deep_ep.EventOverlap()
    ran = []
    ev.register_hook_after_wait(lambda: ran.append(1) or "done")
    assert ev.current_stream_wait() == "done" and ran == [1] and ev.wait() is None
    with ev:
        pass
