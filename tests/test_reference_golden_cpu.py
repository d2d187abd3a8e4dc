"""The all-rank oracle against the golden manifest that the reference checks in (``tests/golden/deepep_reference_v2.json``).

The manifest pins, per case, how many route slots are valid, how many rows every rank receives in the rank layout
(one per token and destination rank) and in the expanded layout (one per token and local expert), and a SHA-256 over
the per-rank, per-local-expert counts.  Its inputs are defined by closed formulas (``tests/utils/cases.py:110-176`` of
the reference: expert ``(11 r + 7 t + 13 s) mod E``, masked when ``(5 r + 3 t + s + 1) mod 97 == 0``), restated here
with tensors.  ``tests/data/reference_golden.json`` holds those four fields of every case.  Agreement means this
library counts, deduplicates and sizes exactly like the reference's own oracle, for 1 to 8 ranks and up to 4096 tokens
per rank.
"""
import hashlib
import json
import os

import pytest
import torch

from deepep_b200.oracle import reference as R

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "data", "reference_golden.json")))["cases"]


def routes_of(case):
    tables = []
    for rank, tokens in enumerate(case["tokens_per_rank"]):
        t = torch.arange(tokens).view(-1, 1)
        s = torch.arange(case["topk"]).view(1, -1)
        expert = (rank * 11 + t * 7 + s * 13) % case["experts"]
        masked = (rank * 5 + t * 3 + s + 1) % 97 == 0
        tables.append(torch.where(masked, torch.full_like(expert, -1), expert).to(torch.int64))
    return tables


@pytest.mark.parametrize("case", GOLDEN, ids=[c["name"] for c in GOLDEN])
def test_oracle_matches_the_reference_manifest(case):
    idx = routes_of(case)
    assert sum(int((t >= 0).sum()) for t in idx) == case["valid_route_slots"]
    # the formulas never repeat an expert inside a token, so the two libraries' rules for repeats do not come into play
    for t in idx:
        ordered = torch.sort(t, dim=1).values
        assert not bool(((ordered[:, 1:] == ordered[:, :-1]) & (ordered[:, 1:] >= 0)).any())
    ranked = R.build_layouts(idx, case["experts"], do_expand=False)
    expanded = R.build_layouts(idx, case["experts"], do_expand=True)
    assert [lay.num_rows for lay in ranked] == case["ordinary_rows"]
    assert [lay.num_rows for lay in expanded] == case["expanded_rows"]
    counts = [[int(v) for v in lay.expert_counts.tolist()] for lay in expanded]
    assert counts == [[int(v) for v in lay.expert_counts.tolist()] for lay in ranked]
    digest = hashlib.sha256(json.dumps(counts, ensure_ascii=True, separators=(",", ":")).encode("ascii")).hexdigest()
    assert digest == case["expert_counts_sha256"]
    # and the expanded rows are in the order the reference sorts them: (local expert, source rank, source token, slot)
    for dst, lay in enumerate(expanded):
        local = case["experts"] // case["world_size"]
        expert = torch.stack([idx[int(s)][int(t), int(k)] for s, t, k in zip(lay.row_source[:64], lay.row_token[:64], lay.row_slot[:64])]) \
            if lay.num_rows else torch.zeros(0, dtype=torch.int64)
        keys = [(int(e), int(s), int(t), int(k)) for e, s, t, k in zip(expert, lay.row_source[:64], lay.row_token[:64], lay.row_slot[:64])]
        assert keys == sorted(keys) and all(dst * local <= e < (dst + 1) * local for e, _, _, _ in keys)
