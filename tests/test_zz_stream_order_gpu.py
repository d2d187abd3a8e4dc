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


def test_two_live_buffers_in_one_process():
    """A prefill buffer and a decode buffer alive at the same time, their calls interleaved (each has its own workspace,
    control block and communication stream); a handle of one is refused by the other.  Parity: the reference's
    multi-buffer tests (``tests/clos/source/test_multi_buffer.py``)."""
    import deepep_b200 as deep_ep

    dev = torch.device("cuda")
    H, E, K = 512, 16, 4
    big = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=400, hidden=H, num_topk=K, explicitly_destroy=True)
    small = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=64, hidden=H, num_topk=K, explicitly_destroy=True)
    xs, idxs, ws = {}, {}, {}
    for name, tokens, seed in (("big", 333, 1), ("small", 48, 2)):
        xs[name] = torch.randn((tokens, H), generator=torch.Generator().manual_seed(seed)).bfloat16()
        idxs[name], ws[name] = group_limited_routes(tokens, E, K, 4, 2, seed=seed), make_weights(tokens, K, seed)
    rb, _, _, hb, _ = big.dispatch(xs["big"].to(dev), topk_idx=idxs["big"].to(dev), topk_weights=ws["big"].to(dev), num_experts=E,
                                   do_expand=True)
    rs, _, rws, hs, _ = small.dispatch(xs["small"].to(dev), topk_idx=idxs["small"].to(dev), topk_weights=ws["small"].to(dev),
                                       num_experts=E)                                    # decode buffer: low-latency path
    assert hs.is_low_latency and not hb.is_low_latency
    ref_b, lay_b = R.dispatch([xs["big"]], [idxs["big"]], [ws["big"]], E, do_expand=True)
    ref_s, lay_s = R.dispatch([xs["small"]], [idxs["small"]], [ws["small"]], E, do_expand=True)
    assert bits_equal(rb, ref_b[0][0]) and bits_equal(rs, ref_s[0][0])
    with pytest.raises(ValueError, match="another buffer"):
        small.combine(rs, hb)
    out_s, _, _ = small.combine(rs, hs)
    out_b, _, _ = big.combine(rb, hb)
    assert bits_equal(out_b, R.combine([ref_b[0][0]], lay_b, [333], K)[0][0])
    assert bits_equal(out_s, R.low_latency_combine([ref_s[0][0]], lay_s, [ws["small"]], [48])[0])
    again = big.dispatch(xs["big"].to(dev), handle=hb)[0]
    assert bits_equal(again, rb)
    small.destroy()
    out_b2, _, _ = big.combine(rb, hb)                  # the other buffer is unaffected by its neighbour's teardown
    assert bits_equal(out_b2, out_b)
    big.destroy()


def test_dispatch_and_combine_under_inference_mode():
    """The serving configuration: every call under ``torch.inference_mode`` (tensors without version counters), on the
    high-throughput and on the low-latency path, against the oracle."""
    import deepep_b200 as deep_ep

    dev = torch.device("cuda")
    H, E, K = 512, 16, 4
    big = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=300, hidden=H, num_topk=K, explicitly_destroy=True)
    small = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=64, hidden=H, num_topk=K, explicitly_destroy=True)
    x = torch.randn((200, H), generator=torch.Generator().manual_seed(21)).bfloat16()
    idx, w = group_limited_routes(200, E, K, 4, 2, seed=8), make_weights(200, K, 3)
    ref, lays = R.dispatch([x], [idx], [w], E, do_expand=True)
    sref, slays = R.dispatch([x[:40]], [idx[:40]], [w[:40]], E, do_expand=True)
    with torch.inference_mode():
        xd, idxd, wd = x.to(dev), idx.to(dev), w.to(dev)
        assert idxd.is_inference()
        rx, _, rw, handle, _ = big.dispatch(xd, topk_idx=idxd, topk_weights=wd, num_experts=E, do_expand=True)
        assert handle.topk_idx is not idxd and bits_equal(rx, ref[0][0]) and bits_equal(rw, ref[0][2])
        out, _, _ = big.combine(rx, handle)
        assert bits_equal(out, R.combine([ref[0][0]], lays, [200], K)[0][0])
        idxd.fill_(-1)                                                  # the handle owns a copy of the indices
        assert bits_equal(big.dispatch(xd, handle=handle)[0], rx)
        xs, idxs, ws = x[:40].to(dev), idx[:40].to(dev), w[:40].to(dev)
        rs, _, _, hs, _ = small.dispatch(xs, topk_idx=idxs, topk_weights=ws, num_experts=E)
        assert hs.is_low_latency and bits_equal(rs, sref[0][0])
        outs, _, _ = small.combine(rs, hs)
        assert bits_equal(outs, R.low_latency_combine([sref[0][0]], slays, [w[:40]], [40])[0])
    small.destroy()
    big.destroy()


def test_shared_and_user_communication_streams():
    """``comm_stream="global"`` puts two buffers on the one stream of the process and GPU; a stream of the caller's is
    used as given; the default stays a stream per buffer.  Results against the oracle on each."""
    import deepep_b200 as deep_ep
    from deepep_b200.buffer import get_global_comm_stream

    dev = torch.device("cuda")
    T, H, E, K = 300, 512, 16, 4
    x = torch.randn((T, H), generator=torch.Generator().manual_seed(4)).bfloat16()
    idx, w = group_limited_routes(T, E, K, 4, 2, seed=6), make_weights(T, K, 2)
    ref, lays = R.dispatch([x], [idx], [w], E, do_expand=True)
    want = R.combine([ref[0][0]], lays, [T], K)[0][0]
    mine = torch.cuda.Stream()
    shape = dict(num_max_tokens_per_rank=T, hidden=H, num_topk=K, explicitly_destroy=True)
    a = deep_ep.ElasticBuffer(None, comm_stream="global", **shape)
    b = deep_ep.ElasticBuffer(None, comm_stream="global", **shape)
    c = deep_ep.ElasticBuffer(None, comm_stream=mine, **shape)
    d = deep_ep.ElasticBuffer(None, **shape)
    shared = get_global_comm_stream()
    assert a.get_comm_stream() == shared and b.get_comm_stream() == shared and c.get_comm_stream() == mine
    assert d.get_comm_stream() != shared and d.get_comm_stream() != mine
    xd, idxd, wd = x.to(dev), idx.to(dev), w.to(dev)
    for buf in (a, b, c, d):
        rx, _, _, handle, event = buf.dispatch(xd, topk_idx=idxd, topk_weights=wd, num_experts=E, do_expand=True,
                                               async_with_compute_stream=True)
        event.current_stream_wait()
        assert bits_equal(rx, ref[0][0])
        out, _, _ = buf.combine(rx, handle)
        assert bits_equal(out, want)
    torch.cuda.synchronize()
    for buf in (a, b, c, d):
        buf.destroy()
    assert get_global_comm_stream() == shared                # outlives the buffers that used it
