"""Pure-CPU all-rank reference implementations (ordering, numerics, MegaMoE math)."""
from . import reference

__all__ = ["reference"]
