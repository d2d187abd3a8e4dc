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
                          os.path.join(ROOT, "benchmarks", "configs", "smoke.json"), "--results-dir", str(tmp_path)],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["status"] == "measured" and rec["correctness_result"] == "passed" and rec["statistics"]["iterations"] == 3
    assert len(os.listdir(tmp_path)) == 1


def test_reference_arm_reports_unavailable():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                          "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-1000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and "\n" not in line["unavailable"]
