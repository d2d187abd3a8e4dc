"""The benchmark's command-line contract that needs no GPU: the reference arm answers with one JSON line and exit code 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                          "--warmup", "1"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-500:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "Ascend" in line["unavailable"] and "\n" not in line["unavailable"]


def test_clock_sampler_reads_what_nvidia_smi_prints(tmp_path, monkeypatch):
    """The ``clocks`` entry of the benchmark line: median SM clock under load, the maximum clock and the throttle reasons
    that were active, from a query-only ``nvidia-smi`` loop.  A stand-in program on PATH prints what the tool prints."""
    import os
    import stat
    import sys
    import time

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    import bench

    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/sh\n"
                    "echo '0, 1965, 1965, 410.5, 0x0000000000000004, Not Active, Not Active, Not Active, Active'\n"
                    "echo '0, 1410, 1965, 990.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active'\n"
                    "echo '0, 1395, 1965, 995.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active'\n"
                    "echo 'garbage line'\n"
                    "sleep 5\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    sampler = bench.ClockSampler(0)
    sampler.start()
    time.sleep(0.5)
    got = sampler.stop()
    assert got == {"sm_mhz": 1410.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
    assert all(field.startswith(("index", "clocks", "power.draw")) for field in bench.ClockSampler.QUERY.split(","))   # reads only
    monkeypatch.setenv("PATH", str(tmp_path / "nowhere"))
    absent = bench.ClockSampler(0)
    absent.start()
    assert absent.stop()["reasons"] == ["nvidia-smi unavailable"]
