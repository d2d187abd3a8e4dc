"""The scripts under ``examples/`` run as documented (here: one process each, CPU engine) and report success."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script", ["dispatch_combine.py", "mega_moe.py"])
def test_example_runs(script):
    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    res = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script)], capture_output=True, text=True, timeout=240, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    assert res.stdout.strip().endswith(": ok") and "rank 0/1 on cpu" in res.stdout
