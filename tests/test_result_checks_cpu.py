"""The order-independent result checkers accept every legal schedule and reject each kind of injected damage.
Parity: ``tests/test_reference.py:119-177`` of the reference (checkers against injected faults)."""
import pytest
import torch

from deepep_b200.oracle import checks as C
from deepep_b200.oracle import reference as R
from helpers import make_routes, make_weights

WORLD, T, H, E, K = 2, [20, 13], 64, 8, 3


def _case(expand, fp8=False, align=1):
    xs = [torch.randn((T[r], H if not fp8 else 128), generator=torch.Generator().manual_seed(r)).bfloat16() for r in range(WORLD)]
    idx = [make_routes("invalid", T[r], E, K, WORLD, 40 + r) for r in range(WORLD)]
    ws = [make_weights(T[r], K, r) for r in range(WORLD)]
    outs, lays = R.dispatch(xs, idx, ws, E, do_expand=expand, expert_alignment=align, quantize_fp8=fp8)
    return xs, idx, ws, outs, lays


def _clone(entry):
    x, i, w = entry
    x = tuple(t.clone() for t in x) if isinstance(x, tuple) else x.clone()
    return x, (None if i is None else i.clone()), (None if w is None else w.clone())


@pytest.mark.parametrize("expand,fp8,align", [(True, False, 1), (True, False, 8), (False, False, 1), (True, True, 1)])
def test_any_order_within_a_segment_is_accepted(expand, fp8, align):
    _, _, _, outs, lays = _case(expand, fp8, align)
    for rank in range(WORLD):
        x, i, w = _clone(outs[rank])
        C.check_dispatch(x, i, w, outs[rank], lays[rank])
        for _, rows in C.segments(lays[rank]):               # a different schedule: every segment reversed
            if rows.numel() > 1:
                back = rows.flip(0)
                for t in (x if isinstance(x, tuple) else (x,)) + tuple(v for v in (i, w) if v is not None):
                    t[rows] = t[back].clone()
        C.check_dispatch(x, i, w, outs[rank], lays[rank])
        if align > 1:                                          # padding rows are nobody's business
            pad = torch.ones(lays[rank].num_rows, dtype=torch.bool)
            for _, rows in C.segments(lays[rank]):
                pad[rows] = False
            x[pad] = 7.0
            C.check_dispatch(x, i, w, outs[rank], lays[rank])


@pytest.mark.parametrize("fault", ["drop", "duplicate", "wrong_segment", "weight", "truncate", "channel"])
@pytest.mark.parametrize("expand", [True, False])
def test_injected_damage_is_reported(fault, expand):
    _, _, _, outs, lays = _case(expand)
    want, lay = outs[0], lays[0]
    x, i, w = _clone(want)
    segs = [rows for _, rows in C.segments(lay) if rows.numel() > 1]
    a, b = int(segs[0][0]), int(segs[0][1])
    other = int(segs[1][0])
    if fault == "drop":
        x[a] = 0
    elif fault == "duplicate":
        x[a] = x[b]
    elif fault == "wrong_segment":                             # two rows trade places across segments
        for t in (x, w) + ((i,) if i is not None else ()):
            keep = t[a].clone()
            t[a] = t[other]
            t[other] = keep
    elif fault == "weight":
        w[a] = w[a] + 1.0
    elif fault == "truncate":
        x = x[:-1]
    elif fault == "channel":
        w = None
    with pytest.raises(C.ResultMismatch) as err:
        C.check_dispatch(x, i, w, want, lay)
    text = str(err.value)
    assert {"drop": "missing", "duplicate": "missing", "wrong_segment": "missing", "weight": "metadata", "truncate": "rows:",
            "channel": "weights: missing"}[fault] in text


def test_combine_checker():
    xs, idx, ws, outs, lays = _case(True)
    combined = R.combine([o[0] for o in outs], lays, T, K)
    for rank in range(WORLD):
        want = combined[rank][0]
        C.check_combine(want.clone(), want)
        off = want.clone()
        off[3, 5] = off[3, 5] + off[3, 5].abs() * 0.01 + 0.01
        with pytest.raises(C.ResultMismatch, match="token 3"):
            C.check_combine(off, want)
        C.check_combine(off, want, tolerance=0.1)
        with pytest.raises(C.ResultMismatch, match="shape"):
            C.check_combine(want[:-1], want)
