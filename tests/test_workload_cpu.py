"""Benchmark workload configurations, byte accounting, result records and the config-driven benchmark on the CPU engine."""
import json
import os
import subprocess
import sys

import pytest
import torch

from deepep_b200.utils import workload as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_validation_and_fingerprint():
    cfg = W.WorkloadConfig.from_dict({"world_size": 2, "tokens_per_rank": [5, 0], "experts": 8, "topk": 2})
    assert cfg.fingerprint() == W.WorkloadConfig.from_dict(cfg.to_dict()).fingerprint()
    assert cfg.fingerprint() != W.WorkloadConfig.from_dict({**cfg.to_dict(), "seed": 1}).fingerprint()
    for bad in ({"operation": "scatter"}, {"world_size": 3, "tokens_per_rank": [1, 1, 1], "experts": 8}, {"hidden": 200},
                {"tokens_per_rank": [1, 2]}, {"topk": 9, "experts": 8}, {"unknown": 1}, {"alignment": 16, "layout": "rank"},
                {"operation": "combine", "dispatch_mode": "fresh"}, {"with_weights": 1}, {"tokens_per_rank": [0]}):
        with pytest.raises(ValueError):
            W.WorkloadConfig.from_dict(bad)


def test_every_shipped_config_is_valid():
    folder = os.path.join(ROOT, "benchmarks", "configs")
    names = sorted(os.listdir(folder))
    assert "smoke.json" in names
    from deepep_b200.models.mega_tools import load_model_config

    for name in names:       # two kinds of files: fused-MoE model configurations (mega_*.json) and dispatch / combine workloads
        if name.startswith("mega_"):
            load_model_config(os.path.join(folder, name))
        else:
            W.WorkloadConfig.from_json(os.path.join(folder, name))


def test_duplicate_keys_are_rejected(tmp_path):
    p = tmp_path / "dup.json"
    p.write_text('{"hidden": 256, "hidden": 512}')
    with pytest.raises(ValueError, match="duplicate"):
        W.WorkloadConfig.from_json(str(p))


@pytest.mark.parametrize("route", ["balanced", "skew", "masked", "grouped"])
def test_routes_are_deterministic_and_legal(route):
    cfg = W.WorkloadConfig.from_dict({"world_size": 2, "tokens_per_rank": [33, 7], "experts": 16, "topk": 4, "route": route})
    for rank in range(2):
        idx, w = W.make_routes(cfg, rank)
        idx2, _ = W.make_routes(cfg, rank)
        assert torch.equal(idx, idx2) and idx.shape == (cfg.tokens_per_rank[rank], 4) and w.shape == idx.shape
        assert int(idx.max()) < 16 and int(idx.min()) >= -1
        for row in idx.tolist():
            real = [e for e in row if e >= 0]
            assert len(set(real)) == len(real)


def test_traffic_counts_one_row_per_token_and_destination():
    cfg = W.WorkloadConfig.from_dict({"world_size": 2, "tokens_per_rank": [2, 1], "experts": 4, "topk": 2, "hidden": 128,
                                      "operation": "roundtrip"})
    routes = [torch.tensor([[0, 1], [1, 2]]), torch.tensor([[3, -1]])]       # rows: 1 + 2 + 1
    t = W.traffic(cfg, routes)
    assert t["rank_rows"] == 4 and t["effective_bytes"] == 4 * 128 * 2 * 2
    fp8 = W.WorkloadConfig.from_dict({**cfg.to_dict(), "dtype": "fp8", "operation": "dispatch"})
    assert W.traffic(fp8, routes)["effective_bytes"] == 4 * (128 + 4)


def test_records_and_result_files(tmp_path):
    cfg = W.WorkloadConfig.from_dict({"world_size": 2, "tokens_per_rank": [4, 4], "iterations": 3})
    rec = W.plan(cfg)
    assert rec["status"] == "planned" and rec["schema_version"] == W.SCHEMA_VERSION
    done = W.complete(rec, [[10.0, 20.0, 30.0], [15.0, 5.0, 31.0]], 3.1e6, "passed")
    assert done["statistics"]["mean_rank_max_us"] == pytest.approx((15 + 20 + 31) / 3) and done["statistics"]["p95_us"] == 31.0
    assert done["bandwidth_gbps"] == pytest.approx(3.1e6 / (22.0 * 1000))
    with pytest.raises(ValueError):
        W.complete(rec, [[1.0, 2.0, 3.0]], 1.0, "passed")
    a = W.write_result(str(tmp_path), done)
    b = W.write_result(str(tmp_path), done)
    assert a != b and json.load(open(a))["config_fingerprint"] == cfg.fingerprint()


def test_config_driven_benchmark_runs_on_the_cpu_engine(tmp_path):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", "bench_ep.py"), "--config",
                          os.path.join(ROOT, "benchmarks", "configs", "smoke.json"), "--results-dir", str(tmp_path / "records"),
                          "--csv", str(tmp_path / "summary.csv"), "--baseline-us", "1000"],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["status"] == "measured" and rec["correctness_result"] == "passed" and rec["statistics"]["iterations"] == 3
    stored = os.listdir(tmp_path / "records")
    assert len(stored) == 1
    W.verify_record(json.load(open(tmp_path / "records" / stored[0])))
    lines = (tmp_path / "summary.csv").read_text().splitlines()
    assert len(lines) == 2 and lines[0].split(",") == list(W.CSV_FIELDS) and lines[1].split(",")[-1] != ""


def test_reference_arm_reports_unavailable():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                          "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-1000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and "\n" not in line["unavailable"]


def _measured(cfg, samples, nbytes=3.0e6):
    return W.complete(W.plan(cfg), samples, nbytes, "passed")


def test_a_record_is_checked_against_its_own_samples():
    cfg = W.WorkloadConfig.from_dict({"world_size": 2, "tokens_per_rank": [4, 4], "iterations": 2, "warmup": 0})
    rec = _measured(cfg, [[10.0, 20.0], [20.0, 40.0]])
    assert W.verify_record(rec)["mean_rank_max_us"] == 30.0
    for change in ({"statistics": {**rec["statistics"], "mean_rank_max_us": 1.0}}, {"bandwidth_gbps": 1e9},
                   {"rank_samples_us": [[10.0, 20.0]]}, {"config_fingerprint": "0" * 64}, {"status": "planned"},
                   {"config": {**rec["config"], "iterations": 0}}):
        with pytest.raises(ValueError):
            W.verify_record({**rec, **change})
    # no logical traffic is a bandwidth of zero, not a missing latency
    empty = _measured(cfg, [[1.0, 1.0], [2.0, 2.0]], nbytes=0.0)
    assert empty["bandwidth_gbps"] == 0 and W.verify_record(empty)["mean_rank_max_us"] == 2.0


def test_summary_csv_has_one_row_and_optional_speedup():
    import csv
    import io

    cfg = W.WorkloadConfig.from_dict({"world_size": 2, "tokens_per_rank": [4, 4], "iterations": 2, "warmup": 0})
    rec = _measured(cfg, [[10.0, 20.0], [20.0, 40.0]])
    rows = list(csv.DictReader(io.StringIO(W.summary_csv(rec))))
    assert len(rows) == 1 and set(rows[0]) == set(W.CSV_FIELDS)
    assert rows[0]["latency_mean_us"] == "30.0" and rows[0]["baseline_latency_us"] == rows[0]["speedup"] == ""
    assert rows[0]["tokens_per_rank"] == "4 4" and rows[0]["config_fingerprint"] == cfg.fingerprint()
    with_base = list(csv.DictReader(io.StringIO(W.summary_csv(rec, baseline_latency_us=60.0))))[0]
    assert float(with_base["speedup"]) == 2.0
    assert W.summary_csv(rec, header=False).count("\n") == 1
    with pytest.raises(ValueError):
        W.summary_csv(rec, baseline_latency_us=0.0)


def test_overrides_are_validated_like_the_file():
    cfg = W.WorkloadConfig.from_dict({"world_size": 2, "tokens_per_rank": [4, 4]})
    changed = W.with_overrides(cfg, ["iterations=50", "route=skew", "with_weights=false", "tokens_per_rank=[8, 0]"])
    assert (changed.iterations, changed.route, changed.with_weights, changed.tokens_per_rank) == (50, "skew", False, (8, 0))
    assert changed.fingerprint() != cfg.fingerprint() and W.with_overrides(cfg, []) == cfg
    for bad in (["iterations"], ["speed=3"], ["iterations=0"], ["route=uphill"]):
        with pytest.raises(ValueError):
            W.with_overrides(cfg, bad)


def test_dry_run_plans_without_measuring(tmp_path):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, os.path.join(ROOT, "benchmarks", "bench_ep.py"), "--config",
           os.path.join(ROOT, "benchmarks", "configs", "smoke.json"), "--dry-run", "--set", "iterations=7", "--results-dir", str(tmp_path)]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["status"] == "planned" and rec["config"]["iterations"] == 7 and "statistics" not in rec
    assert os.listdir(tmp_path) == ["plan.json"]
    again = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)        # a plan is never overwritten
    assert again.returncode != 0 and "FileExistsError" in again.stderr


def test_matrix_is_the_product_of_its_axes_without_repeats():
    cfg = W.WorkloadConfig.from_dict({"world_size": 2, "tokens_per_rank": [4, 4]})
    cases = W.expand_matrix(cfg, ['route=["balanced", "skew"]', "hidden=[256, 512, 256]", "tokens_per_rank=[[4, 4], [8, 0]]"])
    assert len(cases) == 2 * 2 * 2 and len({c.fingerprint() for c in cases}) == 8
    assert [c.hidden for c in cases[:4]] == [256, 256, 256, 256] and cases[0].route == "balanced" and cases[1].tokens_per_rank == (8, 0)
    assert W.expand_matrix(cfg, []) == [cfg]
    for bad in (["route"], ["route=skew"], ["route=[]"], ["speed=[1]"], ["hidden=[256]", "hidden=[512]"]):
        with pytest.raises(ValueError, match="matrix axis"):
            W.expand_matrix(cfg, bad)
    with pytest.raises(ValueError, match="matrix member .*hidden"):
        W.expand_matrix(cfg, ["hidden=[256, 200]"])
    with pytest.raises(ValueError, match="at most"):
        W.expand_matrix(cfg, ["seed=" + json.dumps(list(range(100))), "iterations=" + json.dumps(list(range(1, 101)))])


def test_matrix_run_writes_one_record_per_case(tmp_path):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", "bench_ep.py"), "--config",
                          os.path.join(ROOT, "benchmarks", "configs", "smoke.json"), "--matrix", 'layout=["expanded", "rank"]',
                          "--matrix", "hidden=[128, 256]", "--csv", str(tmp_path / "all.csv")],
                         capture_output=True, text=True, env=env, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    records = [json.loads(line) for line in out.stdout.strip().splitlines()]
    assert len(records) == 4 and all(r["correctness_result"] == "passed" for r in records)
    assert {(r["config"]["layout"], r["config"]["hidden"]) for r in records} == {("expanded", 128), ("expanded", 256), ("rank", 128), ("rank", 256)}
    assert len((tmp_path / "all.csv").read_text().splitlines()) == 5          # one header, four rows
