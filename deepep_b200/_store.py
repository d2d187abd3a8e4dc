"""``deep_ep._store``: the reference's import path of :class:`StoreGroup` (``deep_ep/_store.py`` there); the
implementation lives in :mod:`deepep_b200.parallel.store`."""
from .parallel.store import StoreAborted, StoreGroup

__all__ = ["StoreAborted", "StoreGroup"]
