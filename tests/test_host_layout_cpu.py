"""Host functions of the native headers compiled with plain g++ (no nvcc, no GPU) and checked against their Python
mirrors: workspace layouts, the low-latency region, the MegaMoE input block and the tensor-memory scale-chunk offsets.

Parity: the reference compiles ``static``/``constexpr`` functions out of its kernel headers with g++ to test tilings
and layouts bit-exactly (``tests/utils/cpp.py:1-52``, used by ``tests/elastic/test_dispatch.py:1143``).
"""
import json
import os
import shutil
import subprocess

import pytest
import torch

from deepep_b200.parallel import layout as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_INCLUDE = "/usr/local/cuda/include"

SOURCE = r"""
#include <cstdio>
#include "kernels/ws_layout.h"
#include "kernels/ll_api.h"
#include "kernels/mega_route.cuh"
using namespace dep;
int main() {
  const int shapes[][4] = {{1, 64, 256, 2}, {2, 128, 512, 4}, {4, 4096, 7168, 8}, {8, 4096, 7168, 8}, {8, 16384, 4096, 6}, {8, 256, 7168, 8}};
  std::printf("[");
  for (int i = 0; i < 6; ++i) {
    const int P = shapes[i][0], T = shapes[i][1], H = shapes[i][2], K = shapes[i][3];
    const long long ll = T <= 256 ? ll_region_bytes(P, T, K, H) : 0;
    WsLayout w = make_layout(P, T, H, K, ll, 0);
    LLLayout l = make_ll_layout(P, T < 256 ? T : 256, K, H);
    MegaInput m = mega_input_layout(T, H, K);
    std::printf("%s{\"shape\": [%d, %d, %d, %d], \"total\": %lld, \"stage\": %lld, \"partial\": %lld, \"disp_flag\": %lld, \"comb_flag\": %lld, "
                "\"ll\": %lld, \"ll_bank\": %lld, \"ll_ret\": %lld, \"ll_msg\": %d, \"mega_total\": %lld, \"mega_w\": %lld, \"groups\": %d}",
                i ? ", " : "", P, T, H, K, w.total, w.stage, w.partial, w.disp_flag, w.comb_flag, w.ll, l.bank_bytes, l.ret, l.msg_bytes,
                m.total, m.w, (T + kGroupTokens - 1) / kGroupTokens);
  }
  std::printf("]\n");
  // scale-chunk offsets: a permutation of the bytes of every 512-byte chunk
  long long seen = 0, bad = 0;
  for (long long r = 0; r < 256; ++r)
    for (long long k = 0; k < 512; k += 32) {
      const long long o = sf_offset(r, k, 512);
      bad += (o < 0 || o >= 2 * 4 * 512);
      seen += o;
    }
  std::printf("%lld %lld\n", bad, seen);
  return 0;
}
"""


@pytest.fixture(scope="module")
def host_output(tmp_path_factory):
    if shutil.which("g++") is None or not os.path.exists(os.path.join(CUDA_INCLUDE, "cuda_runtime.h")):
        pytest.skip("needs g++ and the CUDA headers")
    d = tmp_path_factory.mktemp("host")
    src, exe = d / "layouts.cpp", d / "layouts"
    src.write_text(SOURCE)
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "deepep_b200", "csrc"), "-I", CUDA_INCLUDE, str(src), "-o", str(exe)],
                   check=True, capture_output=True, text=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines()
    return json.loads(out[0]), [int(v) for v in out[1].split()]


def test_workspace_layouts_match_the_python_mirror(host_output):
    rows, _ = host_output
    for row in rows:
        P, T, H, K = row["shape"]
        ll = L.ll_region_bytes(P, T, H, K)
        assert row["ll"] and ll == 2 * row["ll_bank"] if T <= 256 else ll == 0
        assert row["total"] == L.workspace_bytes(P, T, H, K, ll)
        assert row["total"] % L.ALIGN == 0 and row["stage"] % 1024 == 0 and row["partial"] > row["stage"]
        # one 8-byte flag per (rank, group of four tokens), dispatch and combine
        assert row["comb_flag"] - row["disp_flag"] == L.align_up(P * row["groups"] * 8, 1024)
        assert row["ll_msg"] == L.align_up(H * 2, 128)
        assert row["mega_total"] % 1024 == 0 and row["mega_w"] < row["mega_total"]


def test_scale_chunk_offsets_are_a_permutation(host_output):
    _, (bad, seen) = host_output
    n = 256 * 16                                       # 256 rows x 16 scale bytes: two row blocks x four K blocks of 512 bytes
    assert bad == 0 and seen == n * (n - 1) // 2       # every byte offset 0..n-1 exactly once


def test_native_layout_equals_host_layout():
    """The pybind layout (what kernels get) is the same function the host test compiled."""
    from deepep_b200.ops import load_native

    C = load_native(build_if_missing=True)
    lay = C.make_layout(8, 4096, 7168, 8, 0, 0)
    assert lay.total == L.workspace_bytes(8, 4096, 7168, 8, 0) and lay.comb_flag > lay.disp_flag > lay.wret
