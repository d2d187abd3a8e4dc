"""Fused-MoE tooling on the CPU: preflight, metrics, golden cache, experimental import names."""
import pytest
import torch

from deepep_b200.models import mega_tools as T


def test_check_routing():
    T.check_routing([[0, 3], [2, -1]], [[0.5, 0.5], [1.0, 0.0]], 4, 2)
    with pytest.raises(ValueError, match="duplicate"):
        T.check_routing([[1, 1]], [[0.5, 0.5]], 4, 2)
    with pytest.raises(ValueError, match="expert ids"):
        T.check_routing([[0, 4]], [[0.5, 0.5]], 4, 2)
    with pytest.raises(ValueError, match="expert ids"):
        T.check_routing([[0, -1]], [[0.5, 0.5]], 4, 2, allow_masked=False)
    with pytest.raises(ValueError, match="finite"):
        T.check_routing([[0, 1]], [[0.5, float("nan")]], 4, 2)
    with pytest.raises(ValueError, match="top-k"):
        T.check_routing([[0]], [[0.5]], 4, 2)


def test_collective_check():
    class Fake:
        def __init__(self, replies):
            self.replies = replies

        def all_gather_object(self, obj):
            return self.replies

    T.collective_check(Fake([(None, 1), (None, 1)]), "inputs", None, 1)
    with pytest.raises(ValueError, match="rank=1: boom"):
        T.collective_check(Fake([(None, 1), ("boom", 1)]), "inputs", None, 1)
    with pytest.raises(ValueError, match="disagree"):
        T.collective_check(Fake([(None, 1), (None, 2)]), "inputs", None, 1)


def test_metrics_and_gate():
    e = torch.tensor([0.0, 2.0, -4.0, 100.0])
    a = torch.tensor([0.001, 2.0, -4.2, 101.0])
    m = T.error_metrics(a, e)
    assert m["max_abs"] == pytest.approx(1.0) and m["mare"] == pytest.approx(0.05) and m["nonfinite"] == 0.0
    assert m["rmse"] == pytest.approx(((0.001 ** 2 + 0.2 ** 2 + 1.0) / 4) ** 0.5, rel=1e-4)
    assert T.compare(a, e, pct_thd=0.5)["ok"] and not T.compare(a, e, pct_thd=0.1)["ok"]
    assert not T.compare(torch.tensor([float("nan")]), torch.tensor([1.0]))["ok"]
    assert not T.compare(torch.tensor([1.2]), torch.tensor([1.0]))["ok"]       # beyond max_diff


def test_golden_cache_roundtrip(tmp_path):
    spec = T.contract(world=2, tokens=[5, 3], hidden=128, intermediate=128, experts=4, topk=2, seed=1)
    assert T.digest(spec) == T.digest(dict(spec)) != T.digest({**spec, "seed": 2})
    first = T.generate(spec, str(tmp_path))
    assert len(list(tmp_path.iterdir())) == 2
    again = T.generate(spec, str(tmp_path))            # served from the cache
    for a, b in zip(first, again):
        assert torch.equal(a, b)
    ok, rows = T.accuracy_report(first, spec, str(tmp_path))
    assert ok and all(r["mare"] == 0.0 for r in rows)
    ok, _ = T.accuracy_report([f + 1 for f in first], spec, str(tmp_path))
    assert not ok


def test_experimental_import_names():
    import deep_ep_experimental.ep_gmm_fused as gmm
    import deep_ep_experimental.megamoe as mega
    from deep_ep_experimental.ep_gmm_fused import alltoallv_gmm, gmm_alltoallv, grouped_matmul_all_to_allv

    assert gmm.all_to_allv_grouped_matmul is alltoallv_gmm and grouped_matmul_all_to_allv is gmm_alltoallv
    assert hasattr(mega, "fp8_fp4_mega_moe") and hasattr(mega, "SymmBuffer") and hasattr(mega, "transform_weights_for_mega_moe")


def test_alias_package_shares_module_objects():
    import deep_ep.parallel.elastic as alias_elastic
    import deep_ep.utils.math as alias_math
    import deepep_b200.parallel.elastic as elastic
    import deepep_b200.utils.math as real_math

    assert alias_math is real_math and alias_elastic is elastic     # one module object, one class identity
    import deep_ep

    assert deep_ep.ElasticBuffer is elastic.ElasticBuffer


def test_model_configurations_in_the_reference_schema(tmp_path):
    """The shipped model configurations load; malformed ones are refused with the reason."""
    import glob
    import json
    import os

    import pytest

    from deepep_b200.models import mega_tools as MT

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "configs")
    shipped = sorted(glob.glob(os.path.join(root, "mega_*.json")))
    assert len(shipped) == 3
    for path in shipped:
        cfg = MT.load_model_config(path)
        assert set(cfg["model"]) == set(MT.MODEL_FIELDS) and cfg["bs_values"] and cfg["iters"] >= 1
    pro = MT.load_model_config(os.path.join(root, "mega_deepseek_v4_pro_shared1.json"))["model"]
    assert pro == dict(hidden=7168, intermediate_hidden=3072, num_experts=384, num_topk=6, num_shared_experts=1)
    good = dict(schema_version=1, model=dict(hidden=256, intermediate_hidden=128, num_experts=4, num_topk=2, num_shared_experts=1),
                bs_values=[3])

    def load(**changes):
        doc = json.loads(json.dumps(good))
        for key, value in changes.items():
            if key in doc["model"]:
                doc["model"][key] = value
            elif value is None:
                doc.pop(key)
            else:
                doc[key] = value
        path = tmp_path / "c.json"
        path.write_text(json.dumps(doc))
        return MT.load_model_config(str(path))

    assert load() == dict(good, warmup=3, iters=10, seed=0)
    for changes, message in ((dict(schema_version=2), "schema_version 1"), (dict(extra=1), "unknown configuration fields: extra"),
                             (dict(hidden=200), "multiple of 256"), (dict(intermediate_hidden=100), "multiple of 256"),
                             (dict(num_topk=5), "num_topk"), (dict(num_shared_experts=15), "at most 16"),
                             (dict(bs_values=[]), "non-empty"), (dict(bs_values=[0]), "batch sizes"), (dict(iters=0), "iters"),
                             (dict(model={"hidden": 256}), "exactly")):
        with pytest.raises(ValueError, match=message):
            load(**changes)


def test_config_driven_benchmark_on_the_cpu_engine(tmp_path):
    """``benchmarks/bench_mega_config.py`` end to end without a GPU: a small model with a shared expert, checked against the
    restatement, one JSON line on stdout."""
    import json
    import os
    import subprocess
    import sys

    import pytest
    import torch

    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = tmp_path / "tiny.json"
    path.write_text(json.dumps(dict(schema_version=1, bs_values=[2, 5], warmup=0, iters=1, seed=3,
                                    model=dict(hidden=256, intermediate_hidden=128, num_experts=4, num_topk=2, num_shared_experts=1))))
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    res = subprocess.run([sys.executable, os.path.join(root, "benchmarks", "bench_mega_config.py"), "--config", str(path), "--check"],
                         capture_output=True, text=True, timeout=240, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    out = json.loads(res.stdout.strip().splitlines()[-1])
    assert out["engine"] == "cpu" and out["world"] == 1 and [r["bs"] for r in out["results"]] == [2, 5]
    assert all(r["ok"] and r["us"] > 0 for r in out["results"])
