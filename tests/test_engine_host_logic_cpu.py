"""Host-side logic of the CUDA engine with a recording stand-in for the native module (no GPU): how blocks are divided
between the NVLink side and the local side, worst-case row capacities, and the passes of a combine whose workspace
holds the partials of a token window only.  Parity: the reference tests its host ops against a fake native module
(``tests/runtime/test_runtime.py``)."""
import types

import pytest
import torch

from deepep_b200.parallel import engine_cuda as EC


def make_engine(world=4, n=1, sm_count=148, max_tokens=1024, partial_tokens=1024, topk=8, hidden=256, local_direct=True):
    calls = []

    class Native:
        def combine(self, lay, sessions, args, send, recv, stream, local_direct, profile, begin, end):
            calls.append(dict(send=send, recv=recv, begin=begin, end=end, ranks=len(args), local_direct=local_direct))

    eng = object.__new__(EC.CudaEngine)
    eng.C, eng.sessions, eng.n, eng.world, eng.sm_count = Native(), [object()] * n, n, world, sm_count
    eng.device = torch.device("cpu")
    eng.layout = types.SimpleNamespace(world=world, max_tokens=max_tokens, partial_tokens=partial_tokens, topk=topk, hidden=hidden)
    eng.default_blocks = eng.combine_blocks = eng.dispatch_blocks = max(2, min(sm_count // n, sm_count - 4))
    eng.combine_send_fraction = EC.COMBINE_SEND_FRACTION.get(world, 0.6)
    eng.dispatch_send_fraction = EC.DISPATCH_SEND_FRACTION.get(world, 0.35)
    eng.local_direct, eng._profile, eng._device_profile, eng._prof, eng._timings = local_direct, False, False, {}, []
    eng._stream = lambda stream=None: 0
    return eng, calls


def plan_for(tokens, rows, topk=8):
    z = torch.zeros(4, dtype=torch.int32)
    return types.SimpleNamespace(num_tokens=tokens, stage_meta=z, rank_rows=z, rank_tokens=z, send_slot=z,
                                 topk_idx=torch.zeros(4, dtype=torch.int64), meta_stride=10, num_experts=16, expand=True, num_rows=rows)


def test_block_division():
    eng, _ = make_engine(world=8)
    assert eng.split_blocks(0, 0.35) == (50, 94)                       # default budget: all but four SMs
    assert eng.split_blocks(64, 0.5) == (32, 32) and eng.split_blocks(3, 0.99) == (2, 1) and eng.split_blocks(2, 0.0) == (1, 1)
    assert eng.split_blocks(10_000, 0.6) == (89, 59)                   # a request above the device is cut to it
    one, _ = make_engine(world=1)
    assert one.split_blocks(100, 1.0) == (100, 0) and one.split_blocks(100, 0.0) == (0, 100)     # one rank, direct local rows
    staged, _ = make_engine(world=1, local_direct=False)
    assert staged.split_blocks(100, 1.0) == (99, 1)                    # rows go through the staging area: both sides needed


def test_worst_case_row_capacity():
    eng, _ = make_engine(world=4, max_tokens=1000, topk=8)
    assert eng.row_capacity(16, 1, True) == 4 * 1000 * 4               # four local experts bound the copies of a token
    assert eng.row_capacity(256, 1, True) == 4 * 1000 * 8
    assert eng.row_capacity(256, 128, True) == 4 * 1000 * 8 + 64 * 127  # every local expert may need a full pad
    assert eng.row_capacity(256, 1, False) == 4 * 1000                 # rank layout: one row per (source, token)


def test_combine_runs_one_pass_per_token_window():
    # real ranks cannot see each other's batch sizes: every rank runs every pass of the capped workspace
    eng, calls = make_engine(world=4, n=1, max_tokens=1024, partial_tokens=256)
    x = torch.zeros((8, 256), dtype=torch.bfloat16)
    out = eng.combine([x], [plan_for(300, 8)], [None])
    assert [(c["begin"], c["end"]) for c in calls] == [(0, 256), (256, 512), (512, 768), (768, 1024)]
    assert out[0][0].shape == (300, 256) and out[0][1] is None and all(c["send"] + c["recv"] == 144 for c in calls)
    # virtual ranks share one launch and know all batch sizes: passes stop at the largest batch
    eng, calls = make_engine(world=2, n=2, max_tokens=1024, partial_tokens=256)
    eng.combine([x, x], [plan_for(300, 8), plan_for(10, 8)], [None, None])
    assert [(c["begin"], c["end"]) for c in calls] == [(0, 256), (256, 512)] and calls[0]["ranks"] == 2
    # a workspace that holds all partials: one pass
    eng, calls = make_engine(world=4, n=1, max_tokens=1024, partial_tokens=1024)
    w = torch.zeros((8,), dtype=torch.float32)
    out = eng.combine([x], [plan_for(0, 8)], [w], split=(40, 24))
    assert [(c["begin"], c["end"], c["send"], c["recv"]) for c in calls] == [(0, 1024, 40, 24)] and out[0][1].shape == (0, 8)
    with pytest.raises(ValueError, match="must not exceed 148"):
        eng.combine([x], [plan_for(4, 8)], [None], split=(100, 60))


def test_status_block_becomes_a_readable_error():
    class Session:
        def __init__(self, **status):
            self._status = dict(code=0, op=0, rank=0, peer=0, where=0, expected=0, seen=0, **status) if not status else status

        def status(self):
            return self._status

    eng = object.__new__(EC.CudaEngine)
    eng.sessions = [Session()]
    eng.check_status()                                                     # code 0: nothing to report
    eng.sessions = [Session(), Session(code=1, op=3, rank=5, peer=2, where=1, expected=7, seen=6)]
    with pytest.raises(EC.CommunicationError, match=r"rank 5: combine timeout at wait site 1 \(the partial sums of an expert rank\) on "
                                                     r"peer 2 \(expected 7, saw 6\); restart"):
        eng.check_status()
    eng.sessions = [Session(code=2, op=2, rank=0, peer=-1, where=103, expected=10, seen=12)]
    with pytest.raises(EC.CommunicationError, match=r"dispatch bad argument at wait site 103 on peer -1"):
        eng.check_status()
    assert all(op in EC.OP_NAMES for op, _ in EC.WAIT_SITES)


def test_argument_keys_agree_between_python_and_the_bindings():
    """The engine hands every kernel its arguments as a dict; the bindings read the keys they know and treat a missing one
    as null / zero.  A misspelt key would therefore go unnoticed until a kernel dereferences the null: the two key sets
    must be equal for every operation."""
    import ast
    import os
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def cpp_keys(path, func):
        src = open(os.path.join(root, "deepep_b200", "csrc", path)).read()
        start = src.index("{", src.index(func + "("))
        depth, at = 0, start
        while True:
            depth += {"{": 1, "}": -1}.get(src[at], 0)
            if depth == 0:
                break
            at += 1
        body = src[start:at]
        return set(re.findall(r'\(d, "([A-Za-z0-9_]+)"', body)) | set(re.findall(r'd\["([A-Za-z0-9_]+)"\]', body))

    tree = ast.parse(open(os.path.join(root, "deepep_b200", "parallel", "engine_cuda.py")).read())
    methods = {f.name: f for n in ast.walk(tree) if isinstance(n, ast.ClassDef) and n.name == "CudaEngine"
               for f in n.body if isinstance(f, ast.FunctionDef)}

    def py_keys(method):
        keys = set()
        for call in ast.walk(methods[method]):
            if isinstance(call, ast.Call) and getattr(call.func, "attr", None) == "append" and call.args \
                    and isinstance(call.args[0], ast.Call) and getattr(call.args[0].func, "id", None) == "dict":
                keys |= {k.arg for k in call.args[0].keywords}
        return keys

    for func, path, method in (("op_notify", "bindings.cpp", "notify"), ("op_dispatch", "bindings.cpp", "dispatch"),
                               ("op_combine", "bindings.cpp", "combine"), ("op_ll_dispatch", "ll_bindings.cpp", "ll_dispatch"),
                               ("op_ll_combine", "ll_bindings.cpp", "ll_combine")):
        native, python = cpp_keys(path, func), py_keys(method)
        assert python and native == python, (func, sorted(python - native), sorted(native - python))
