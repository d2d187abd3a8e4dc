"""The public classes against the reference's machine-readable API contract.

``tests/data/api_contract.json`` holds, per public object and method, the parameter names, kinds and defaults that the
reference pins in ``tests/api/api_contract.json`` (checked there by ``tests/api/test_contracts.py``).  Every contract
method must exist here, accept every contract parameter by the same name, keep the order of the positional ones, and
use the same default unless the deviation is listed below with its reason.
"""
import inspect
import json
import os

import pytest

import deepep_b200 as deep_ep

CONTRACT = json.load(open(os.path.join(os.path.dirname(__file__), "data", "api_contract.json")))

# (object, method, parameter) -> reason; empty: every default equals the contract's
DEVIATIONS = {}


def _methods():
    for oname, methods in CONTRACT["objects"].items():
        for mname, spec in methods.items():
            yield oname, mname, spec


def test_exports_resolve_lazily():
    for name in CONTRACT["exports"]:
        assert getattr(deep_ep, name) is not None
    for name in ("topk_idx_t", "Handle", "Slot", "SlotState", "ExpandHandle"):
        assert getattr(deep_ep, name) is not None


@pytest.mark.parametrize("oname,mname,spec", list(_methods()), ids=lambda v: v if isinstance(v, str) else "")
def test_method_matches_contract(oname, mname, spec):
    cls = getattr(deep_ep, oname)
    assert hasattr(cls, mname), f"{oname}.{mname} is missing"
    raw = inspect.getattr_static(cls, mname)
    if spec["kind"] == "staticmethod":
        assert isinstance(raw, staticmethod) or not inspect.signature(getattr(cls, mname)).parameters.get("self"), \
            f"{oname}.{mname} must be callable without an instance"
    sig = inspect.signature(getattr(cls, mname))
    have = sig.parameters
    accepts_any = any(p.kind is inspect.Parameter.VAR_KEYWORD for p in have.values())
    names = list(have)
    last = -1
    for entry in spec["parameters"]:
        name, kind = entry[0], entry[1]
        if name == "self":
            continue
        if name not in have:
            assert accepts_any, f"{oname}.{mname} does not accept {name!r}"
            continue
        if kind == "POSITIONAL_OR_KEYWORD" and have[name].kind is inspect.Parameter.POSITIONAL_OR_KEYWORD:
            assert names.index(name) > last, f"{oname}.{mname}: positional order of {name!r} differs"
            last = names.index(name)
        if len(entry) == 3 and (oname, mname, name) not in DEVIATIONS:
            assert have[name].default == entry[2], f"{oname}.{mname}({name}): default {have[name].default!r}, contract {entry[2]!r}"


def test_deviations_are_real():
    """Every listed deviation names an existing parameter whose default really differs (no stale entries)."""
    for (oname, mname, pname), reason in DEVIATIONS.items():
        assert reason
        spec = {e[0]: e for e in CONTRACT["objects"][oname][mname]["parameters"]}
        have = inspect.signature(getattr(getattr(deep_ep, oname), mname)).parameters
        assert pname in spec and pname in have
        assert len(spec[pname]) == 3 and have[pname].default != spec[pname][2], (oname, mname, pname)
