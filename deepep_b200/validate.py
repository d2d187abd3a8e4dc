"""Installation check: ``python -m deepep_b200.validate [--package-only]``.

Two parts, the counterparts of the reference's ``scripts/validate_package.py`` (what an installed package must contain
and how it must behave at import) and ``scripts/validate_ep.py`` (an expert-parallel smoke run through the public API):

* package: importing ``deepep_b200`` / ``deep_ep`` loads neither torch nor the native extension; the lazy names
  resolve; the native binary is the one its provenance file describes and speaks the expected runtime protocol;
* smoke: one process dispatches to identity experts and combines, in the expanded and in the rank layout, on the GPU
  when there is one (native kernels) and through the CPU engine otherwise; results must equal ``sum_k w_k * x``.  Then
  one tiny fused MoE forward and one ``alltoallv_gmm`` call, each against its restatement.

Prints one JSON object and exits non-zero when a check fails.
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys


def check_package() -> dict:
    out = {}
    code = ("import sys, deepep_b200, deep_ep; "
            "print(int('torch' in sys.modules), int('deepep_b200._C' in sys.modules), deep_ep.ElasticBuffer.__name__)")
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    fields = res.stdout.split()
    out["import_is_lazy"] = res.returncode == 0 and fields[:2] == ["0", "0"] and fields[2:] == ["ElasticBuffer"]
    from .ops import build_info, load_native, native_path

    out["binary_present"] = native_path().exists()
    info = build_info()
    out["build_info"] = {k: info.get(k) for k in ("arch", "nvcc", "runtime_protocol", "debug_bounds", "binary")}
    try:
        mod = load_native()
        out["native_loads"], out["runtime_protocol"] = True, int(mod.runtime_protocol)
        out["capabilities"] = info.get("capabilities", [])
    except Exception as exc:          # reported, not raised: the JSON tells what is wrong
        out["native_loads"], out["error"] = False, str(exc)
    out["ok"] = bool(out["import_is_lazy"] and out["binary_present"] and out["native_loads"] and info.get("arch") == "sm_100a")
    return out


def smoke() -> dict:
    import torch

    from . import ElasticBuffer

    cuda = torch.cuda.is_available()
    dev = torch.device("cuda") if cuda else torch.device("cpu")
    T, H, E, K = 96, 512, 8, 4
    g = torch.Generator().manual_seed(0)
    x = torch.randn((T, H), generator=g).bfloat16().to(dev)
    idx = torch.rand((T, E), generator=g).topk(K, dim=1).indices.to(torch.int64).to(dev)
    w = torch.softmax(torch.randn((T, K), generator=g), dim=1).to(dev)
    buf = ElasticBuffer(None, num_max_tokens_per_rank=512, hidden=H, num_topk=K, explicitly_destroy=True)
    out = {"engine": "cuda" if cuda else "cpu"}
    try:
        rx, _, rw, h, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, do_expand=True)
        y, _, _ = buf.combine((rx.float() * rw.unsqueeze(1)).bfloat16(), h)
        want = x.float() * w.sum(1, keepdim=True)
        out["expanded_layout"] = bool(torch.allclose(y.float(), want, rtol=0.02, atol=0.06))
        rx2, ridx, _, h2, _ = buf.dispatch(x, topk_idx=idx, num_experts=E, do_expand=False)
        y2, _, _ = buf.combine(rx2, h2)
        out["rank_layout"] = bool(torch.equal(rx2, x) and torch.allclose(y2.float(), x.float(), rtol=0.01, atol=0.03))
    finally:
        buf.destroy()
    out["fused_moe"] = _smoke_fused_moe(dev)
    out["alltoallv_gmm"] = _smoke_gmm(dev, g)
    out["ok"] = bool(out.get("expanded_layout") and out.get("rank_layout") and out["fused_moe"] and out["alltoallv_gmm"])
    return out


def _smoke_fused_moe(dev) -> bool:
    """The fused MoE layer on one rank against its CPU restatement (tcgen05 kernel on a GPU, CPU engine otherwise)."""
    import torch

    from .models import mega_tools as MT
    from .models.mega_moe import SymmBuffer, fp8_fp4_mega_moe, transform_weights_for_mega_moe

    spec = MT.contract(world=1, tokens=[48], hidden=512, intermediate=256, experts=4, topk=2, seed=3)
    xs, idx, ws, l1, l2 = MT.make_case(spec)
    sym = SymmBuffer(None, 4, 64, 2, 512, 256)
    try:
        w1, w2 = transform_weights_for_mega_moe(l1, l2, device=dev)
        sym.load_inputs(xs[0][0].to(dev), xs[0][1].to(dev), idx[0].to(dev), ws[0].to(dev))
        y = torch.zeros((48, 512), dtype=torch.bfloat16, device=dev)
        fp8_fp4_mega_moe(y, w1, w2, sym, check=dev.type == "cuda")
        ok, _ = MT.accuracy_report([y.cpu()], spec)
        return bool(ok)
    finally:
        sym.destroy()


def _smoke_gmm(dev, g) -> bool:
    """``alltoallv_gmm`` on one rank against an fp32 matmul of the same rows."""
    import torch

    from .ops import ep_gmm_fused as G

    counts = [40, 0, 70, 18]
    x = torch.randn((sum(counts), 128), generator=g).bfloat16()
    w = (torch.randn((4, 128, 128), generator=g) / 11).bfloat16()
    G.init_group(None, max_rows=256, max_k=128, max_n=128)
    try:
        out = G.alltoallv_gmm(x.to(dev), w.to(dev), counts, counts, ep_size=1, expert_num=4)
        if dev.type == "cuda":
            torch.cuda.synchronize()
        ref, _ = G.reference_alltoallv_gmm([x], [w], [counts], 4)
        return bool(torch.allclose(out.float().cpu(), ref[0].float(), rtol=0.03, atol=0.03))
    finally:
        G.destroy_group()


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--package-only", action="store_true", help="skip the dispatch/combine smoke run")
    args = ap.parse_args()
    report = {"package": check_package()}
    if not args.package_only:
        report["smoke"] = smoke()
    report["ok"] = all(part["ok"] for part in report.values() if isinstance(part, dict))
    print(json.dumps(report, indent=1))
    return 0 if report["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
