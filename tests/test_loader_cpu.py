"""The loader of the native extension under faults made on the host: a binary that is missing, one that speaks another
runtime protocol, one whose import fails, and what ``require_native`` tells the caller in each case.
Parity: ``tests/runtime/test_loader.py`` of the reference."""
import types

import pytest

import deepep_b200.ops as ops


@pytest.fixture
def fresh(monkeypatch):
    monkeypatch.setattr(ops, "_native", None)
    return monkeypatch


def test_missing_binary_names_the_build_command(fresh, tmp_path):
    fresh.setattr(ops, "native_path", lambda: tmp_path / "_C.missing.so")
    with pytest.raises(ops.NativeUnavailable, match=r"is not built; run `python -m deepep_b200._build`"):
        ops.load_native()
    with pytest.raises(NotImplementedError, match="ElasticBuffer needs the native CUDA extension"):
        ops.require_native("ElasticBuffer")
    assert ops.native_available() is False


def test_another_runtime_protocol_is_refused(fresh):
    fresh.setattr(ops, "_verify_binary", lambda: None)
    fresh.setattr(ops.importlib, "import_module", lambda name: types.SimpleNamespace(runtime_protocol=ops.RUNTIME_PROTOCOL + 1))
    with pytest.raises(ops.NativeUnavailable, match="another runtime protocol"):
        ops.load_native()
    assert ops._native is None                                   # nothing half-loaded is kept


def test_import_failure_is_reported_with_its_reason(fresh):
    def broken(name):
        raise ImportError("libcudart.so.12: cannot open shared object file")

    fresh.setattr(ops, "_verify_binary", lambda: None)
    fresh.setattr(ops.importlib, "import_module", broken)
    with pytest.raises(ops.NativeUnavailable, match="failed to load: libcudart"):
        ops.require_native("MegaMoE")


def test_provenance_is_optional_but_binding_when_present(fresh):
    fresh.setattr(ops, "build_info", lambda: {})                 # no provenance file: nothing to compare with
    ops._verify_binary()
    fresh.setattr(ops, "build_info", lambda: {"binary": "some_other_name.so", "binary_sha256": "0" * 64})
    with pytest.raises(ops.NativeUnavailable, match="not the one"):
        ops._verify_binary()


def test_loaded_module_is_cached(fresh):
    calls = []
    module = types.SimpleNamespace(runtime_protocol=ops.RUNTIME_PROTOCOL)

    def importer(name):
        calls.append(name)
        return module

    fresh.setattr(ops, "_verify_binary", lambda: None)
    fresh.setattr(ops.importlib, "import_module", importer)
    assert ops.load_native() is module and ops.load_native() is module and calls == ["deepep_b200._C"]
    assert ops.require_native("anything") is module and ops.native_available()
