"""Machine detection and the cross-rank consensus rules that run when a buffer is constructed (no GPU needed: the
rules are applied to reports, and the reports of GPU ranks are written by hand)."""
import pytest
import torch

from deepep_b200.parallel import topology as T


def _gpu(rank, device, **kw):
    base = dict(rank=rank, host="node0", kind="nvswitch", device=device, uuid=f"GPU-{device}", name="NVIDIA B200",
                capability=(10, 0), sm_count=148, visible=4, peer_access={d: True for d in range(4)})
    base.update(kw)
    return T.RankMachine(**base)


def test_detect_without_gpu_reports_cpu():
    m = T.detect(3, None)
    assert m.kind == "cpu" and m.rank == 3 and m.host
    assert T.check_consensus([m, T.detect(4, torch.device("cpu"))]) == "cpu"


def test_consensus_accepts_one_nvswitch_domain():
    assert T.check_consensus([_gpu(r, r) for r in range(4)]) == "nvswitch"
    assert T.check_consensus([_gpu(0, 2)]) == "single"
    assert T.check_consensus([_gpu(r, r) for r in range(2)], "nvswitch") == "nvswitch"
    assert T.check_consensus([_gpu(0, 0)], "b200") == "single"          # one rank of an NVSwitch machine


@pytest.mark.parametrize("reports, message", [
    ([_gpu(0, 0), T.RankMachine(rank=1, host="node0", kind="cpu")], "some ranks run on GPUs"),
    ([_gpu(0, 0), _gpu(1, 1, host="node1")], "one NVLink domain"),
    ([_gpu(0, 0), _gpu(1, 1, name="NVIDIA H100", capability=(9, 0))], "different GPUs"),
    ([_gpu(0, 0, name="NVIDIA H100", capability=(9, 0)), _gpu(1, 1, name="NVIDIA H100", capability=(9, 0))], "capability 10"),
    ([_gpu(0, 1), _gpu(1, 1)], "same GPU"),
    ([_gpu(0, 0, peer_access={0: True, 1: False}), _gpu(1, 1)], "no peer access"),
])
def test_consensus_rejects(reports, message):
    with pytest.raises(RuntimeError, match=message):
        T.check_consensus(reports)


def test_requested_machine_type_must_match():
    with pytest.raises(RuntimeError, match="requested"):
        T.check_consensus([T.detect(0, None)], "nvswitch")
    with pytest.raises(ValueError):
        T.check_consensus([_gpu(0, 0)], "mesh")
    assert T.check_consensus([T.detect(0, None)], "cpu") == "cpu"


def test_buffer_records_the_agreed_machine():
    from deepep_b200 import ElasticBuffer

    buf = ElasticBuffer(None, num_max_tokens_per_rank=16, hidden=128, num_topk=2, explicitly_destroy=True, device="cpu")
    assert buf.machine_type == "cpu"
    buf.destroy()
    with pytest.raises(RuntimeError, match="requested"):
        ElasticBuffer(None, num_max_tokens_per_rank=16, hidden=128, num_topk=2, explicitly_destroy=True, device="cpu",
                      machine_type="nvswitch")


def test_probe_command_reports_and_decides(capsys, monkeypatch):
    """``python -m deepep_b200.parallel.topology``: prints the reports as JSON; the exit code says whether the planned
    ranks would pass the constructor's check."""
    import json

    import torch

    from deepep_b200.parallel import topology as TP

    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert TP.main(["--ranks", "3"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["ok"] and out["machine_type"] == "cpu" and out["ranks"] == 3 and len(out["reports"]) == 3
    # two planned ranks on a machine with one GPU: the check refuses (one GPU per rank)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 1)
    monkeypatch.setattr(TP, "detect", lambda rank, device=None: TP.RankMachine(
        rank=rank, host="h", kind="single", device=0, uuid="GPU-1", name="NVIDIA B200", capability=(10, 0), sm_count=148,
        visible=1, peer_access={0: True}))
    assert TP.main(["--ranks", "2"]) == 1
    out = json.loads(capsys.readouterr().out)
    assert not out["ok"] and "same GPU" in out["error"]
    assert TP.main([]) == 0 and json.loads(capsys.readouterr().out)["machine_type"] == "single"


def test_buffers_report_their_machine_selection():
    """``buffer.machine_type`` / ``buffer.machine_selection`` (the reference prints both after construction): what was asked
    for, what all ranks agreed on, and every rank's report."""
    import deepep_b200 as deep_ep

    buf = deep_ep.ElasticBuffer(None, num_max_tokens_per_rank=8, hidden=64, num_topk=2, device="cpu", machine_type="cpu")
    try:
        sel = buf.machine_selection
        assert buf.machine_type == "cpu" == sel["machine_type"] and sel["requested"] == "cpu"
        assert [r["rank"] for r in sel["ranks"]] == [0] and sel["ranks"][0]["kind"] == "cpu"
    finally:
        buf.destroy()
    lazy = deep_ep.Buffer(None)
    assert lazy.machine_type is None and lazy.machine_selection is None        # no workspace yet
    sized = deep_ep.Buffer(None, num_max_tokens_per_rank=8, hidden=64, num_topk=2)
    assert sized.machine_type == "cpu" and sized.machine_selection["machine_type"] == "cpu"
    sized.destroy()
