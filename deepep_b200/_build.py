"""In-tree build of the native extension ``deepep_b200._C`` for sm_100a.

Every ``.cu``/``.cpp`` under ``csrc/`` is compiled with nvcc
(``-gencode arch=compute_100a,code=sm_100a -lineinfo``) into ``csrc/build/`` and
linked into ``deepep_b200/_C<EXT_SUFFIX>`` next to this file, so the binary
travels with the source tree.  Objects are rebuilt only when their source, a
header or the flags changed.  ``python -m deepep_b200._build`` builds from the
command line; ``-v`` adds ``-Xptxas -v``.
"""
from __future__ import annotations

import hashlib
import json
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
BUILD = CSRC / "build"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def target_path() -> Path:
    return ROOT / ("_C" + sysconfig.get_config_var("EXT_SUFFIX"))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (cand == "nvcc" or Path(cand).exists()):
            return cand
    raise RuntimeError("nvcc not found")


def _flags(verbose: bool) -> list:
    import pybind11

    flags = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden",
             "-I", str(CSRC), "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], *ARCH_FLAGS]
    if os.environ.get("DEEPEP_DEBUG_BOUNDS", "0") not in ("", "0"):   # index checks in the kernels (see common.cuh)
        flags += ["-DDEEPEP_DEBUG_BOUNDS"]
    if verbose:
        flags += ["-Xptxas", "-v"]
    return flags


def sources() -> list:
    return sorted(list(CSRC.glob("*.cpp")) + list(CSRC.glob("runtime/*.cpp")) + list(CSRC.glob("kernels/*.cu")))


def _digest(src: Path, flags: list) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(src.read_bytes())
    for hdr in sorted(list(CSRC.glob("**/*.h")) + list(CSRC.glob("**/*.cuh"))):
        h.update(hdr.read_bytes())
    return h.hexdigest()


CAPABILITIES = ["ep_notify", "ep_dispatch_ht", "ep_combine_ht", "ep_dispatch_ll", "ep_combine_ll", "ep_barrier", "ep_expand",
                "ep_aggregate", "mega_moe", "a2av_gmm", "gmm_a2av", "transport:vmm", "transport:ipc"]


def write_build_info(binary: Path, nvcc: str) -> None:
    """Provenance of the binary next to it: what was compiled, with what, and the binary's hash (checked by the loader)."""
    info = {"arch": "sm_100a", "nvcc": subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout.strip().splitlines()[-1],
            "sources": [s.relative_to(ROOT).as_posix() for s in sources()], "runtime_protocol": 1,
            "debug_bounds": os.environ.get("DEEPEP_DEBUG_BOUNDS", "0") not in ("", "0"), "capabilities": CAPABILITIES,
            "binary": binary.name, "binary_sha256": hashlib.sha256(binary.read_bytes()).hexdigest()}
    (ROOT / "_build_info.json").write_text(json.dumps(info, indent=1))


def build(verbose: bool = False, force: bool = False) -> Path:
    BUILD.mkdir(parents=True, exist_ok=True)
    nvcc, flags = _nvcc(), _flags(verbose)
    stamp_file = BUILD / "stamps.json"
    stamps = json.loads(stamp_file.read_text()) if stamp_file.exists() and not force else {}
    jobs, objects = [], []
    for src in sources():
        obj = BUILD / (src.relative_to(CSRC).as_posix().replace("/", "_") + ".o")
        objects.append(obj)
        digest = _digest(src, flags)
        if obj.exists() and stamps.get(obj.name) == digest:
            continue
        jobs.append((src, obj, digest))

    def compile_one(job):
        src, obj, digest = job
        cmd = [nvcc, *flags, "-x", "cu", "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose or res.stderr.strip():
            sys.stderr.write(f"--- {src.name}\n{res.stderr}")
        return obj.name, digest

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for name, digest in pool.map(compile_one, jobs):
                stamps[name] = digest
        stamp_file.write_text(json.dumps(stamps, indent=0))
    out = target_path()
    if jobs or not out.exists() or not (ROOT / "_build_info.json").exists():
        cmd = [nvcc, "-shared", *ARCH_FLAGS, "-o", str(out), *map(str, objects)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        write_build_info(out, nvcc)
    return out


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
