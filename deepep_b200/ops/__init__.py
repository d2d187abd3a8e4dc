"""Loader of the native extension and thin launch helpers.

Parity: ``deep_ep/_native.py:27-46, 114-156`` of the reference (lazy
``require_native``; explicit failure when the extension is missing; protocol
check).  The extension is built in-tree by :mod:`deepep_b200._build`; it is
never rebuilt implicitly at import time on a GPU machine.
"""
from __future__ import annotations

import importlib
import json
from pathlib import Path
from typing import Any, Optional

RUNTIME_PROTOCOL = 1
_native: Optional[Any] = None


class NativeUnavailable(NotImplementedError):
    pass


def native_path() -> Path:
    from .._build import target_path

    return target_path()


def load_native(build_if_missing: bool = False):
    """Import ``deepep_b200._C``; optionally build it first when it does not exist."""
    global _native
    if _native is not None:
        return _native
    if not native_path().exists():
        if not build_if_missing:
            raise NativeUnavailable(
                f"native extension {native_path().name} is not built; run `python -m deepep_b200._build`")
        from .._build import build

        build()
    _verify_binary()
    mod = importlib.import_module("deepep_b200._C")
    if getattr(mod, "runtime_protocol", None) != RUNTIME_PROTOCOL:
        raise NativeUnavailable("native extension speaks another runtime protocol; rebuild it")
    _native = mod
    return mod


def _verify_binary() -> None:
    """When the build left its provenance file, the binary on disk must be the one it describes (a stale or foreign
    ``_C*.so`` is refused instead of being loaded into the process)."""
    info = build_info()
    digest = info.get("binary_sha256")
    if not digest:
        return
    import hashlib

    if info.get("binary") != native_path().name or hashlib.sha256(native_path().read_bytes()).hexdigest() != digest:
        raise NativeUnavailable("the native extension on disk is not the one _build_info.json describes; "
                                "run `python -m deepep_b200._build`")


def require_native(operation: str):
    """Return the extension or raise a NotImplementedError that names the operation."""
    try:
        return load_native()
    except NativeUnavailable as exc:
        raise NativeUnavailable(f"{operation} needs the native CUDA extension: {exc}") from exc
    except ImportError as exc:
        raise NativeUnavailable(f"{operation} needs the native CUDA extension, which failed to load: {exc}") from exc


def native_available() -> bool:
    try:
        load_native()
        return True
    except Exception:
        return False


def build_info() -> dict:
    path = Path(__file__).resolve().parent.parent / "_build_info.json"
    return json.loads(path.read_text()) if path.exists() else {}


__all__ = ["NativeUnavailable", "build_info", "load_native", "native_available", "native_path", "require_native"]
