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
