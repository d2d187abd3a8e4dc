"""Device-side records as Chrome-trace / Perfetto timelines (``deepep_b200/utils/trace.py``): hand-made records of each
kind, checked span by span.  Parity: the reference's trace tooling (``timer/trace_parser.py``, ``notify_profile.py``)."""
import json

import torch

from deepep_b200.utils import trace as TR


def test_phase_stamps_become_consecutive_spans():
    stamps = {"table_sent": 8.0, "tables_in": 9.5, "histograms": 14.0, "never_reached": 0.0, "done": 40.0}
    events = TR.from_phase_stamps("notify", stamps, rank=3, track=1, offset_us=100.0)
    assert [e["name"] for e in events] == ["notify:table_sent", "notify:tables_in", "notify:histograms", "notify:done"]
    assert [(e["ts"], e["dur"]) for e in events] == [(100.0, 8.0), (108.0, 1.5), (109.5, 4.5), (114.0, 26.0)]
    assert all(e["pid"] == 3 and e["tid"] == 1 and e["ph"] == "X" for e in events)


def test_device_profile_blocks_become_threads():
    profile = {("dispatch", 0): [dict(role="sender", start_us=0.0, end_us=30.0, meta_us=1.0, wait_us=2.0, data_us=20.0, publish_us=4.0, rows=64),
                                 dict(role="receiver", start_us=1.0, end_us=35.5, meta_us=0.5, wait_us=25.0, data_us=9.0, publish_us=0.0, rows=70)],
               ("combine", 1): [dict(role="expert", start_us=2.0, end_us=12.0, meta_us=0.0, wait_us=0.0, data_us=9.0, publish_us=1.0, rows=8)]}
    events = TR.from_device_profile(profile, offset_us=10.0)
    assert [(e["name"], e["pid"], e["tid"], e["ts"], e["dur"]) for e in events] == [
        ("combine:expert", 1, 0, 12.0, 10.0), ("dispatch:sender", 0, 0, 10.0, 30.0), ("dispatch:receiver", 0, 1, 11.0, 34.5)]
    assert events[2]["args"] == {"meta_us": 0.5, "wait_us": 25.0, "data_us": 9.0, "publish_us": 0.0, "rows": 70}
    table = TR.summarize(events)
    assert table["dispatch:sender"] == {"count": 1, "total_us": 30.0, "max_us": 30.0, "mean_us": 30.0}


def test_mega_timer_records_become_cta_timelines():
    ns = 1_000_000                                     # %globaltimer counts nanoseconds
    wait_word = (250 << 32) | 1000                     # the MMA thread waited 250 of 1000 (cycles / 16)
    timer = torch.tensor([[ns, ns + 12_000, ns + 30_000, ns + 400_000, ns + 1_400_000, ns + 1_411_000, ns + 1_530_000, wait_word],
                          [0, 0, 0, 0, 0, 0, 0, 0],                                                 # a CTA that did not run
                          [ns + 1_000, ns + 12_500, ns + 30_500, 0, ns + 1_380_000, ns + 1_411_500, ns + 1_520_000, 0]],
                         dtype=torch.int64)
    events = TR.from_mega_timer(timer, rank=2)
    by = {(e["tid"], e["name"]): e for e in events}
    assert by[(0, "mega_moe:handshake")]["ts"] == 0.0 and by[(0, "mega_moe:handshake")]["dur"] == 12.0
    assert by[(0, "mega_moe:gemm")]["ts"] == 30.0 and by[(0, "mega_moe:gemm")]["dur"] == 1370.0
    assert by[(0, "mega_moe:gemm")]["args"] == {"mma_thread_wait_share": 0.25}
    assert by[(1, "mega_moe:pull")]["ts"] == 30.0 and by[(1, "mega_moe:pull")]["dur"] == 370.0      # pull warps: a thread of their own
    assert by[(0, "mega_moe:reduce")]["dur"] == 119.0 and by[(4, "mega_moe:handshake")]["ts"] == 1.0
    assert (5, "mega_moe:pull") not in by and not any(e["tid"] in (2, 3) for e in events)             # no stamp, no span
    assert all(e["pid"] == 2 for e in events) and TR.from_mega_timer(torch.zeros((2, 8), dtype=torch.int64)) == []


def test_written_file_is_a_trace_event_document(tmp_path):
    events = TR.from_phase_stamps("ll_dispatch", {"routes_read": 2.2, "rows_sent": 9.7}, rank=1) \
        + TR.from_phase_stamps("ll_dispatch", {"routes_read": 2.0, "rows_sent": 9.0}, rank=0)
    path = TR.write_trace(str(tmp_path / "t.json"), events, rank_names={0: "GPU 0"})
    doc = json.load(open(path))
    names = [e for e in doc["traceEvents"] if e["ph"] == "M"]
    assert [(e["pid"], e["args"]["name"]) for e in names] == [(0, "GPU 0"), (1, "rank 1")]
    spans = [e for e in doc["traceEvents"] if e["ph"] == "X"]
    assert [e["pid"] for e in spans] == [0, 0, 1, 1] and spans[0]["ts"] <= spans[1]["ts"]
    assert TR.span("late", 5.0, 3.0)["dur"] == 0.0
