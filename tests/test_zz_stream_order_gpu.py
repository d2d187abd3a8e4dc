"""Calls ordered after an event instead of after the current stream (``previous_event``), asynchronous completion and
outputs taken from the communication stream's memory pool (``allocate_on_comm_stream``), against the oracle.

Parity: the stream / event contract of the reference (``docs/api.md:134-142``,
``deep_ep/backends/mesh_clos/elastic.py:958-1008``).  This file sorts late on purpose.
"""
import pytest
import torch

from deepep_b200.oracle import reference as R
from helpers import bits_equal, group_limited_routes, make_weights

pytestmark = pytest.mark.gpu


def test_previous_event_async_and_comm_stream_allocation():
    import deepep_b200 as deep_ep

    dev = torch.device("cuda")
    T, H, E, K = 300, 1024, 32, 6
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(11)).bfloat16()
    idx, w = group_limited_routes(T, E, K, 8, 4, seed=3), make_weights(T, K, 5)
    ref, lays = R.dispatch([x * 2], [idx], [w], E, do_expand=True)
    cref = R.combine([ref[0][0]], lays, [T], K)
    buf = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=T, hidden=H, num_topk=K, explicitly_destroy=True)
    xd, idxd, wd = x.to(dev), idx.to(dev), w.to(dev)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):                      # the input is produced on a side stream ...
        x2 = xd * 2
        produced = deep_ep.EventHandle()               # ... and only this event orders the dispatch after it
    rx, _, rw, handle, event = buf.dispatch(x2, topk_idx=idxd, topk_weights=wd, num_experts=E, do_expand=True,
                                            previous_event=produced, async_with_compute_stream=True,
                                            allocate_on_comm_stream=True)
    assert event.event is not None
    event.current_stream_wait()
    assert bits_equal(rx, ref[0][0]) and bits_equal(rw, ref[0][2])
    # asynchronous combine ordered after an event recorded on the current stream; outputs from the comm stream's pool
    out, _, done = buf.combine(rx, handle, previous_event=deep_ep.EventHandle(), async_with_compute_stream=True)
    with done:                                          # leaving the block makes the current stream wait
        pass
    assert bits_equal(out, cref[0][0])
    # synchronous cached dispatch after an EventOverlap: the result is usable on the current stream at return
    again, _, _, _, ev = buf.dispatch(x2, handle=handle, previous_event=deep_ep.EventOverlap(deep_ep.EventHandle()))
    assert ev.event is None and bits_equal(again, rx)
    torch.cuda.synchronize()
    buf.destroy()
