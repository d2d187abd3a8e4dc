"""Argument validation and handle rules of ``ElasticBuffer`` on the CPU engine (one process): every documented
rejection raises the documented exception and leaves the buffer usable."""
import pytest
import torch

from helpers import make_weights


T, H, K, E = 48, 256, 4, 8


@pytest.fixture()
def buf():
    from deepep_b200 import ElasticBuffer

    b = ElasticBuffer(None, num_max_tokens_per_rank=512, hidden=H, num_topk=K, explicitly_destroy=True, device="cpu")
    yield b
    b.destroy()


def _inputs(tokens=T):
    g = torch.Generator().manual_seed(0)
    x = torch.randn((tokens, H), generator=g).bfloat16()
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(tokens)]).to(torch.int64)
    return x, idx, make_weights(tokens, K)


@pytest.mark.parametrize("kwargs, message", [
    (dict(num_max_tokens_per_rank=0, hidden=H, num_topk=K), "required"),
    (dict(num_max_tokens_per_rank=1 << 20, hidden=H, num_topk=K), "limits"),
    (dict(num_max_tokens_per_rank=64, hidden=H, num_topk=64), "limits"),
    (dict(num_max_tokens_per_rank=64, hidden=H, num_topk=K, machine_type="mesh_clos"), "machine_type"),
    (dict(num_max_tokens_per_rank=64, hidden=H, num_topk=K, bootstrap="mpi"), "bootstrap"),
    (dict(num_max_tokens_per_rank=64, hidden=H, num_topk=K, num_gpu_timeout_secs=0), "seconds"),
    (dict(num_max_tokens_per_rank=64, hidden=100, num_topk=K, use_fp8_dispatch=True), "hidden"),
])
def test_constructor_rejections(kwargs, message):
    from deepep_b200 import ElasticBuffer

    with pytest.raises(ValueError, match=message):
        ElasticBuffer(None, explicitly_destroy=True, device="cpu", **kwargs)


def test_dispatch_rejections_leave_the_buffer_usable(buf):
    x, idx, w = _inputs()
    bad = [
        (dict(x=x[:, :128], topk_idx=idx, num_experts=E), "tokens,"),                       # wrong hidden
        (dict(x=x.t().contiguous().t(), topk_idx=idx, num_experts=E), "contiguous"),
        (dict(x=torch.zeros((600, H), dtype=torch.bfloat16), topk_idx=torch.zeros((600, K), dtype=torch.int64), num_experts=E), "exceed"),
        (dict(x=x.float(), topk_idx=idx, num_experts=E), "bf16"),
        (dict(x=x, topk_idx=idx.int(), num_experts=E), "topk_idx"),
        (dict(x=x, topk_idx=idx[:, :2].contiguous(), num_experts=E), "topk_idx"),
        (dict(x=x, topk_idx=idx, topk_weights=w.double(), num_experts=E), "topk_weights"),
        (dict(x=x, topk_idx=idx, num_experts=0), "num_experts"),
        (dict(x=x, topk_idx=idx, num_experts=2048), "num_experts"),
        (dict(x=x, num_experts=E), "fresh dispatch"),
        (dict(x=x, topk_idx=idx, num_experts=E, expert_alignment=0, do_expand=True), "positive"),
        (dict(x=x, topk_idx=idx, num_experts=E, expert_alignment=16), "do_expand"),
        (dict(x=(x, torch.ones((T, H // 128))), topk_idx=idx, num_experts=E), "fp8 pair"),
    ]
    for kwargs, message in bad:
        xin = kwargs.pop("x")
        with pytest.raises(ValueError, match=message):
            buf.dispatch(xin, **kwargs)
    rx, _, rw, handle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True)   # still fine
    assert rx.shape[0] == T * K and handle.num_recv_tokens_per_expert_list is not None


def test_combine_and_handle_rules(buf):
    from deepep_b200 import ElasticBuffer

    x, idx, w = _inputs()
    rx, _, rw, handle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True)
    with pytest.raises(ValueError, match="rows"):
        buf.combine(rx[:-1], handle)
    with pytest.raises(ValueError, match="bf16"):
        buf.combine(rx.float(), handle)
    with pytest.raises(ValueError, match="contiguous"):
        buf.combine(torch.zeros((H, rx.shape[0]), dtype=torch.bfloat16).t(), handle)
    with pytest.raises(ValueError, match="topk_weights"):
        buf.combine(rx, handle, topk_weights=rw.double())
    with pytest.raises(ValueError, match="bias"):
        buf.combine(rx, handle, bias=torch.zeros((T, H)))
    with pytest.raises(ValueError, match="together"):
        buf.combine(rx, handle, combine_num_sms=8)
    with pytest.raises(ValueError, match="nonnegative"):
        buf.combine(rx, handle, combine_num_sms=-1, reduce_num_sms=4)
    with pytest.raises(TypeError, match="EPHandle"):
        buf.combine(rx, object())
    with pytest.raises(ValueError, match="token count"):
        buf.dispatch(x[:10].contiguous(), handle=handle)
    with pytest.raises(ValueError, match="not both"):
        buf.dispatch(x, topk_idx=idx, num_experts=E, handle=handle)
    other = ElasticBuffer(None, num_max_tokens_per_rank=512, hidden=H, num_topk=K, explicitly_destroy=True, device="cpu")
    try:
        with pytest.raises(ValueError, match="another buffer"):
            other.combine(rx, handle)
    finally:
        other.destroy()
    out, ow, _ = buf.combine(rx, handle, topk_weights=rw)                       # the handle survived all of the above
    assert out.shape == (T, H) and torch.equal(ow, w)
    again = buf.dispatch(x, handle=handle)[0]                                   # cached dispatch re-uses the routing
    assert torch.equal(again.view(torch.int16), rx.view(torch.int16))
    handle.topk_idx[0, 0] = (handle.topk_idx[0, 0] + 1) % E                     # in-place edit of saved routing is detected
    with pytest.raises(RuntimeError, match="modified"):
        buf.combine(rx, handle)


def test_low_latency_selection_rules():
    """A buffer of at most 256 tokens serves a default fresh dispatch with weights on the low-latency path; every option
    that path does not have (``do_expand``, alignment, statistics, an SM budget, a cached handle) selects the other one."""
    from deepep_b200 import ElasticBuffer

    small = ElasticBuffer(None, num_max_tokens_per_rank=64, hidden=H, num_topk=K, explicitly_destroy=True, device="cpu")
    try:
        x, idx, w = _inputs(32)
        assert small.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E)[3].is_low_latency
        assert not small.dispatch(x, topk_idx=idx, num_experts=E)[3].is_low_latency                         # no weights
        assert not small.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True)[3].is_low_latency
        stats = torch.zeros(E, dtype=torch.int64)
        h = small.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, cumulative_local_expert_recv_stats=stats)[3]
        assert not h.is_low_latency and int(stats.sum()) == 32 * K
        assert not small.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, num_sms=24)[3].is_low_latency
        ll = small.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E)
        with pytest.raises(ValueError, match="saved at dispatch"):
            small.combine(ll[0], ll[3], topk_weights=ll[2])
    finally:
        small.destroy()


def test_column_major_scales_and_topology_queries(buf):
    """``use_tma_aligned_col_major_sf`` returns the same scales stored column by column with the row count padded to 4
    (16-byte columns); the sizing queries answer for one NVLink domain."""
    from deepep_b200.utils.math import per_token_cast_to_fp8

    x, idx, w = _inputs(37)
    pair = per_token_cast_to_fp8(x)
    (rx, sf), _, _, handle, _ = buf.dispatch(pair, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True)
    (rx2, sf2), _, _, _, _ = buf.dispatch(pair, handle=handle)
    (rx3, sf3), _, _, _, _ = buf.dispatch(pair, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True,
                                         use_tma_aligned_col_major_sf=True)
    rows = sf.shape[0]
    assert torch.equal(sf, sf2) and torch.equal(sf3, sf) and torch.equal(rx3.view(torch.uint8), rx.view(torch.uint8))
    assert sf.is_contiguous() and sf3.stride() == (1, -(-rows // 4) * 4)
    assert buf.get_physical_domain_size() == (1, 1) and buf.get_logical_domain_size() == (1, 1)
    assert buf.get_theoretical_num_qps(24) == 0
    sms = buf.get_theoretical_num_sms(E, K)
    assert 8 <= sms <= 128 and buf.get_theoretical_num_compute_units(E, K) == sms
    assert buf.pop_profile() == []


def test_a_failed_launch_poisons_the_buffer(buf, monkeypatch):
    """A wait that ran out surfaces as ``CommunicationError``; every later call on the buffer is refused."""
    from deepep_b200.parallel.engine_cuda import CommunicationError

    x, idx, w = _inputs()

    def broken(*a, **k):
        raise CommunicationError("rank 0: dispatch timeout at wait site 1 on peer 0 (expected 3, saw 2)")

    monkeypatch.setattr(buf.engine, "dispatch", broken)
    with pytest.raises(CommunicationError, match="wait site"):
        buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True)
    monkeypatch.undo()
    with pytest.raises(RuntimeError, match="restart the distributed job"):
        buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True)
    with pytest.raises(RuntimeError, match="restart the distributed job"):
        buf.barrier()


def test_calls_under_inference_mode(buf):
    """Serving code runs under ``torch.inference_mode``: tensors made there keep no version counter, so the handle cannot
    watch them for in-place changes and keeps a copy of the indices instead (``do_handle_copy=True``, the default); with
    ``do_handle_copy=False`` the caller's tensor is used as it is.  Parity: ``docs/elastic.md`` of the reference
    ("HT may be called under torch.inference_mode(); an inference tensor as index needs the default do_handle_copy")."""
    import torch

    with torch.inference_mode():
        x, idx, w = _inputs()
        x, idx, w = x.clone(), idx.clone(), w.clone()                       # inference tensors
        assert idx.is_inference()
        rx, _, rw, handle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True)
        assert handle.topk_idx is not idx and torch.equal(handle.topk_idx, idx)
        out, _, _ = buf.combine((rx.float() * rw[:, None]).bfloat16(), handle)
        assert torch.allclose(out.float(), x.float() * w.sum(1, keepdim=True), rtol=0.02, atol=0.03)
        idx.fill_(-1)                                                       # the caller's tensor is free again
        again = buf.dispatch(x, handle=handle)[0]
        assert torch.equal(again, rx)
        x2, idx2, w2 = _inputs()
        idx2 = idx2.clone()
        _, _, _, borrowed, _ = buf.dispatch(x2.clone(), topk_idx=idx2, topk_weights=w2.clone(), num_experts=E, do_expand=True,
                                            do_handle_copy=False)
        assert borrowed.topk_idx is idx2
        rr, ridx, _, h3, _ = buf.dispatch(x2.clone(), topk_idx=idx2, num_experts=E)       # rank layout
        assert torch.equal(buf.combine(rr, h3)[0].float(), x2.float())
    # outside inference mode nothing is copied and changes are detected as before
    x, idx, w = _inputs()
    _, _, _, watched, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True)
    assert watched.topk_idx is idx
    idx[0, 0] = idx[0, 0]
    with pytest.raises(RuntimeError, match="modified in place"):
        buf.dispatch(x, handle=watched)


def test_packed_exponent_scales_travel_bit_for_bit(buf):
    """MXFP8 activations carry four ue8m0 exponents per 128 values packed into an int32 where the fp32 recipe has one
    fp32 scale.  Dispatch moves scale words without touching them, so it accepts either and returns the kind it got."""
    import torch

    g = torch.Generator().manual_seed(9)
    x = torch.randn((20, H), generator=g).to(torch.float8_e4m3fn)
    exponents = torch.randint(100, 140, (20, H // 128, 4), generator=g, dtype=torch.uint8)
    exponents[0, 0] = torch.tensor([255, 255, 192, 0], dtype=torch.uint8)          # a NaN pattern if read as fp32: still copied as is
    sf = exponents.view(torch.int32).view(20, H // 128)
    _, idx, w = _inputs(20)
    (rx, rsf), _, _, handle, _ = buf.dispatch((x, sf), topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True)
    assert rsf.dtype == torch.int32 and rsf.shape == (rx.shape[0], H // 128)
    token = (handle.recv_src_metadata[:rx.shape[0]].long() // K) % buf.num_max_tokens_per_rank
    assert torch.equal(rsf, sf[token]) and torch.equal(rx.view(torch.uint8), x.view(torch.uint8)[token])
    (rx2, rsf2), _, _, _, _ = buf.dispatch((x, sf), handle=handle)
    assert rsf2.dtype == torch.int32 and torch.equal(rsf2, rsf)
    (_, cm), _, _, _, _ = buf.dispatch((x, sf), topk_idx=idx, num_experts=E, do_expand=True, use_tma_aligned_col_major_sf=True)
    assert cm.dtype == torch.int32 and torch.equal(cm, rsf) and cm.stride(0) == 1
    with pytest.raises(ValueError, match="float32 or int32"):
        buf.dispatch((x, sf.to(torch.int64)), topk_idx=idx, num_experts=E)


def test_do_expand_none_means_the_expanded_layout(buf):
    """The reference's fresh dispatch is expanded when ``do_expand`` is not given (``None`` there); upstream's default is
    ``False``.  Both spellings are honoured: the default gives the rank layout, an explicit ``None`` the expanded one."""
    import torch

    x, idx, w = _inputs()
    by_default = buf.dispatch(x, topk_idx=idx, num_experts=E)
    assert by_default[1] is not None and by_default[3].do_expand is False
    as_reference = buf.dispatch(x, topk_idx=idx, num_experts=E, do_expand=None)
    explicit = buf.dispatch(x, topk_idx=idx, num_experts=E, do_expand=True)
    assert as_reference[1] is None and as_reference[3].do_expand is True and torch.equal(as_reference[0], explicit[0])


def test_a_live_handle_keeps_its_buffer():
    """Replacing the variable that held a buffer does not end the buffer while one of its handles is alive; after an
    explicit ``destroy`` the handle is refused."""
    import gc
    import weakref

    from deepep_b200 import ElasticBuffer

    x, idx, w = _inputs()
    first = ElasticBuffer(None, num_max_tokens_per_rank=64, hidden=H, num_topk=K, explicitly_destroy=True, device="cpu")
    rx, _, _, handle, _ = first.dispatch(x, topk_idx=idx, num_experts=E, do_expand=True)
    watcher = weakref.ref(first)
    first = ElasticBuffer(None, num_max_tokens_per_rank=128, hidden=H, num_topk=K, explicitly_destroy=True, device="cpu")
    gc.collect()
    assert watcher() is not None and handle._owner is watcher()
    out, _, _ = watcher().combine(rx, handle)                       # the old buffer still serves its handle
    assert out.shape == x.shape
    with pytest.raises(ValueError, match="another buffer"):
        first.combine(rx, handle)
    watcher().destroy()
    with pytest.raises(RuntimeError, match="destroyed"):
        handle._owner.combine(rx, handle)
    first.destroy()
