"""Block-scaled tcgen05 grouped GEMM (e4m3 x e2m1, ue8m0 per 32) against an fp32 PyTorch reference."""
import pytest
import torch

from deepep_b200.oracle import megamoe as O

pytestmark = pytest.mark.gpu


def _run(rows_per_expert, n_total, k, seed=0, b_tx=None, pair=False, stages=0, commit_every=0):
    from deepep_b200.ops import load_native

    C = load_native()
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(seed)
    experts = len(rows_per_expert)
    tiles = [-(-r // 256) * 2 if pair else -(-r // 128) for r in rows_per_expert]   # CTA pairs: whole pairs of tiles per expert
    rows_pad = 128 * sum(tiles)
    x = torch.randn((rows_pad, k), generator=g)
    a_codes, a_sf = O.quantize_mxfp8(x)
    packed = torch.randint(0, 256, (experts * n_total, k // 2), generator=g, dtype=torch.uint8)
    b_sf = torch.randint(118, 123, (experts * n_total, k // 32), generator=g, dtype=torch.uint8)
    mtile_expert = torch.tensor([e for e, t in enumerate(tiles) for _ in range(t)], dtype=torch.int32)
    ref = torch.empty((rows_pad, n_total))
    a_f, b_f = O.dequantize_mxfp8(a_codes, a_sf), O.unpack_fp4(packed, b_sf)
    for mt, e in enumerate(mtile_expert.tolist()):
        ref[mt * 128:(mt + 1) * 128] = a_f[mt * 128:(mt + 1) * 128] @ b_f[e * n_total:(e + 1) * n_total].t()
    d = dict(a=a_codes.view(torch.uint8).to(dev), b=O.tile_fp4_rows(packed).to(dev), sfa=O.to_sf_chunks(a_sf).to(dev), sfb=O.to_sf_chunks(b_sf).to(dev),
             mt=mtile_expert.to(dev), n=torch.tensor([len(mtile_expert)], dtype=torch.int32, device=dev),
             c=torch.zeros((rows_pad, n_total), dtype=torch.float32, device=dev), err=torch.zeros(1, dtype=torch.int32, device=dev))
    args = dict(a=d["a"].data_ptr(), b=d["b"].data_ptr(), sfa=d["sfa"].data_ptr(), sfb=d["sfb"].data_ptr(),
                mtile_expert=d["mt"].data_ptr(), num_mtiles=d["n"].data_ptr(), rows_pad=rows_pad, k=k, b_rows=experts * n_total,
                n_total=n_total, epi=0, c=d["c"].data_ptr(), ldc=n_total, error_flag=d["err"].data_ptr())
    if b_tx is not None:
        args["b_tx_bytes"] = b_tx
    if pair:
        args["pair"] = 1
    if stages:
        args["stages"] = stages
    if commit_every:
        args["commit_every"] = commit_every
    C.mega_gemm(args, None, 148, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert d["err"].item() == 0, "a pipeline wait ran out inside the GEMM kernel"
    out = d["c"].cpu()
    err = (out - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-3 * scale + 1e-3, f"max abs error {err} (reference scale {scale})"


def test_single_tile():
    _run([128], 256, 128)


def test_k_loop_and_tiles():
    _run([128, 256], 256, 1024)


def test_grouped_shapes():
    _run([100, 1, 300, 128], 512, 2048, seed=3)


def test_cta_pairs_single_pair():
    """One pair of row blocks, one N tile: the smallest case of the cta_group::2 path (two CTAs, M = 256)."""
    _run([256], 256, 128, pair=True)


def test_cta_pairs_grouped_shapes():
    """Several experts (odd tile counts are padded to whole pairs), a K loop longer than the pipeline, several N tiles."""
    _run([100, 1, 300, 256], 512, 2048, seed=3, pair=True)


def test_pipeline_depth_and_commit_grouping():
    """The operand pipeline with other depths and with two stages released per commit gives the same numbers (K loop of
    16 steps, longer than any of the pipelines; plain and CTA-pair kernels)."""
    _run([128, 256], 256, 2048, seed=5, stages=2)
    _run([128, 256], 256, 2048, seed=5, stages=4, commit_every=2)
    _run([256, 512], 512, 2048, seed=6, pair=True, stages=6, commit_every=2)
    _run([256], 256, 2048, seed=7, pair=True, stages=3)
