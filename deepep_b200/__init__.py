"""deepep_b200: expert-parallel dispatch/combine for MoE models on NVIDIA B200 (sm_100a).

Importing the package loads neither torch nor the native extension; the public
names resolve on first use (parity: ``deep_ep/__init__.py:11-25`` of the reference).
"""
__version__ = "0.2.0"

__all__ = ["Buffer", "ElasticBuffer", "EPHandle", "Config", "EventHandle", "EventOverlap"]

_LAZY = {
    "Buffer": ("deepep_b200.buffer", "Buffer"),
    "ElasticBuffer": ("deepep_b200.parallel.elastic", "ElasticBuffer"),
    "EPHandle": ("deepep_b200.parallel.elastic", "EPHandle"),
    "Config": ("deepep_b200.config", "Config"),
    "EventHandle": ("deepep_b200.utils.event", "EventHandle"),
    "EventOverlap": ("deepep_b200.utils.event", "EventOverlap"),
    "topk_idx_t": ("deepep_b200.buffer", "topk_idx_t"),
    "Handle": ("deepep_b200.resources", "Handle"),
    "Slot": ("deepep_b200.resources", "Slot"),
    "SlotState": ("deepep_b200.resources", "SlotState"),
    "ExpandHandle": ("deepep_b200.ops.expand", "ExpandHandle"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib

        module, attr = _LAZY[name]
        value = getattr(importlib.import_module(module), attr)
        globals()[name] = value
        return value
    raise AttributeError(name)
