"""Whether the library's bf16 grouped GEMM (``torch._grouped_mm``) can be used on this machine.

A library kernel that was compiled for another GPU architecture aborts the process that launches it, so the check
runs a tiny problem in a child process once and caches the verdict; multi-rank callers ask one rank and share it.
"""
from __future__ import annotations

import subprocess
import sys
from typing import Optional

import torch

_PROBE = """
import torch
a = torch.randn(96, 64, device='cuda', dtype=torch.bfloat16)
b = torch.randn(3, 64, 32, device='cuda', dtype=torch.bfloat16)
offs = torch.tensor([32, 32, 96], device='cuda', dtype=torch.int32)
out = torch._grouped_mm(a, b, offs=offs)
torch.cuda.synchronize()
ref = torch.cat([a[:32] @ b[0], a[32:32] @ b[1], a[32:] @ b[2]])
assert torch.allclose(out.float(), ref.float(), rtol=0.05, atol=0.5)
"""
_verdict: Optional[bool] = None


def grouped_mm_usable(force: Optional[bool] = None) -> bool:
    """``force`` installs a verdict obtained elsewhere (another rank); otherwise the first call probes."""
    global _verdict
    if force is not None:
        _verdict = bool(force)
    if _verdict is None:
        _verdict = bool(hasattr(torch, "_grouped_mm") and torch.cuda.is_available() and
                        subprocess.run([sys.executable, "-c", _PROBE], capture_output=True, timeout=300).returncode == 0)
    return _verdict


__all__ = ["grouped_mm_usable"]
