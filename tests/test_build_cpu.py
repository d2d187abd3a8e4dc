"""The in-tree build description (no compiler is run): flags, source list, change detection, provenance, and a guard
over every file of the repository for constructs that must never appear in it.

Parity: the reference tests its build configuration without building (``tests/runtime/test_build.py``).
"""
import json
import os
from pathlib import Path

from deepep_b200 import _build as B

REPO = Path(__file__).resolve().parent.parent


def test_flags_name_the_architecture_and_the_switches(monkeypatch):
    monkeypatch.delenv("DEEPEP_DEBUG_BOUNDS", raising=False)
    flags = B._flags(False)
    at = flags.index("-gencode")
    assert flags[at + 1] == "arch=compute_100a,code=sm_100a" and "-lineinfo" in flags and "-std=c++17" in flags
    assert "-DDEEPEP_DEBUG_BOUNDS" not in flags and "-Xptxas" not in flags
    assert B._flags(True)[-2:] == ["-Xptxas", "-v"]
    monkeypatch.setenv("DEEPEP_DEBUG_BOUNDS", "1")
    assert "-DDEEPEP_DEBUG_BOUNDS" in B._flags(False)
    monkeypatch.setenv("DEEPEP_DEBUG_BOUNDS", "0")
    assert "-DDEEPEP_DEBUG_BOUNDS" not in B._flags(False)
    assert B.target_path().parent == Path(B.__file__).resolve().parent and B.target_path().name.startswith("_C")


def test_every_native_source_is_built_and_listed():
    names = {s.relative_to(B.CSRC).as_posix() for s in B.sources()}
    on_disk = {p.relative_to(B.CSRC).as_posix() for p in B.CSRC.rglob("*") if p.suffix in (".cu", ".cpp") and "build" not in p.parts}
    assert names == on_disk and "kernels/ht_dispatch.cu" in names and "runtime/session.cpp" in names and "bindings.cpp" in names
    info_file = Path(B.__file__).resolve().parent / "_build_info.json"
    if info_file.exists():                       # written by the last build: it must describe today's source list
        info = json.loads(info_file.read_text())
        assert info["arch"] == "sm_100a" and info["runtime_protocol"] == 1 and info["capabilities"] == B.CAPABILITIES
        assert set(info["sources"]) == {"csrc/" + n for n in names}


def test_change_detection_sees_flags_sources_and_headers(tmp_path, monkeypatch):
    src = B.CSRC / "kernels" / "barrier.cu"
    base = B._digest(src, ["-O3"])
    assert base == B._digest(src, ["-O3"]) and base != B._digest(src, ["-O2"])
    assert base != B._digest(B.CSRC / "kernels" / "layout.cu", ["-O3"])
    # a header anywhere under csrc/ takes part in every object's digest
    fake = tmp_path / "csrc"
    (fake / "kernels").mkdir(parents=True)
    (fake / "kernels" / "a.cu").write_text("// a\n")
    (fake / "kernels" / "h.cuh").write_text("// one\n")
    monkeypatch.setattr(B, "CSRC", fake)
    first = B._digest(fake / "kernels" / "a.cu", [])
    (fake / "kernels" / "h.cuh").write_text("// two\n")
    assert B._digest(fake / "kernels" / "a.cu", []) != first


def test_compiler_lookup(monkeypatch, tmp_path):
    tool = tmp_path / "my-nvcc"
    tool.write_text("#!/bin/sh\n")
    monkeypatch.setenv("NVCC", str(tool))
    assert B._nvcc() == str(tool)
    monkeypatch.setenv("NVCC", str(tmp_path / "missing"))
    assert B._nvcc() in ("/usr/local/cuda/bin/nvcc", "nvcc")


def _text_files():
    ignored = (REPO / ".gitignore").read_text().split() if (REPO / ".gitignore").exists() else []
    skip = {".git", "__pycache__", "build", ".pytest_cache"} | {entry.strip("/").split("/")[-1] for entry in ignored if entry.endswith("/")}
    for root, dirs, files in os.walk(REPO):
        dirs[:] = [d for d in dirs if d not in skip]
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".h", ".cpp", ".sh", ".json", ".toml", ".cfg")):
                yield Path(root) / name


def test_no_file_names_a_closed_call_or_a_multicast_load():
    """Batched memcpy entry points fault this driver, and a bulk / tensor load with cluster multicast must never reach
    another GPU's memory: no source, script or configuration may name either (comments included)."""
    closed = ["cudaMemcpy" + mid + "Batch" + "Async" for mid in ("", "3D")] + ["cuMemcpy" + mid + "Batch" + "Async" for mid in ("", "3D")]
    bulk, multi = "cp.async" + ".bulk", ".multicast" + "::cluster"
    clock_setters = ("nvidia-smi -" + "lgc", "nvidia-smi -" + "ac", "nvidia-smi -" + "pm", "--lock-gpu-" + "clocks")
    bad = []
    for path in _text_files():
        text = path.read_text(errors="ignore")
        for word in closed + list(clock_setters):
            if word in text:
                bad.append((str(path.relative_to(REPO)), word))
        for number, line in enumerate(text.splitlines(), 1):
            if bulk in line and multi in line:
                bad.append((str(path.relative_to(REPO)), f"line {number}: bulk load with cluster multicast"))
    assert not bad, bad


def test_no_python_module_uses_a_name_it_never_binds():
    """A misspelt or forgotten import only fails when its line runs, which for GPU-only paths is on a GPU: every name a
    module loads must be bound somewhere in it (assignment, definition, import, parameter) or be a builtin."""
    import ast
    import builtins

    known = set(dir(builtins)) | {"__file__", "__name__", "__doc__"}
    bad = {}
    for path in _text_files():
        if path.suffix != ".py":
            continue
        tree = ast.parse(path.read_text())
        bound, loaded, star = set(), {}, False
        for node in ast.walk(tree):
            if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)):
                bound.add(node.name)
            if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef, ast.Lambda)):
                args = node.args
                bound |= {a.arg for a in args.args + args.kwonlyargs + args.posonlyargs}
                bound |= {a.arg for a in (args.vararg, args.kwarg) if a is not None}
            elif isinstance(node, ast.Import):
                bound |= {(a.asname or a.name).split(".")[0] for a in node.names}
            elif isinstance(node, ast.ImportFrom):
                star = star or any(a.name == "*" for a in node.names)
                bound |= {a.asname or a.name for a in node.names}
            elif isinstance(node, ast.Name):
                if isinstance(node.ctx, ast.Load):
                    loaded.setdefault(node.id, node.lineno)
                else:
                    bound.add(node.id)
            elif isinstance(node, ast.ExceptHandler) and node.name:
                bound.add(node.name)
            elif isinstance(node, (ast.Global, ast.Nonlocal)):
                bound |= set(node.names)
        unbound = {name: line for name, line in loaded.items() if name not in bound and name not in known}
        if unbound and not star:
            bad[str(path.relative_to(REPO))] = unbound
    assert not bad, bad


def test_package_metadata_agrees():
    import re

    import deepep_b200

    declared = re.search(r'^version = "([^"]+)"', (REPO / "pyproject.toml").read_text(), re.M).group(1)
    assert deepep_b200.__version__ == declared
    listed = re.search(r"^packages = \[(.*?)\]", (REPO / "pyproject.toml").read_text(), re.M | re.S).group(1)
    for package in ("deepep_b200", "deepep_b200.models", "deepep_b200.ops", "deepep_b200.oracle", "deepep_b200.parallel",
                    "deepep_b200.utils", "deep_ep", "deep_ep_experimental"):
        assert f'"{package}"' in listed and (REPO / package.replace(".", "/") / "__init__.py").exists()
