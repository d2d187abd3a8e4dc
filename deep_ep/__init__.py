"""Drop-in import name: ``import deep_ep`` resolves to :mod:`deepep_b200`.

Code written against the reference (``deep_ep.ElasticBuffer``, ``deep_ep.Buffer``,
``deep_ep.utils...``) keeps working unchanged.
"""
import importlib
import sys

import deepep_b200 as _impl

__all__ = list(_impl.__all__)
__version__ = _impl.__version__


def __getattr__(name):
    return getattr(_impl, name)


class _AliasFinder:
    """Maps ``deep_ep.<sub>`` to ``deepep_b200.<sub>`` (utils, oracle, parallel, models, ...)."""

    @staticmethod
    def find_spec(fullname, path=None, target=None):
        if not fullname.startswith("deep_ep."):
            return None
        real = "deepep_b200." + fullname[len("deep_ep."):]
        try:
            module = importlib.import_module(real)
        except ImportError:
            return None
        # sys.modules[fullname] is set by the import system from what the loader's create_module returns; setting it
        # here would make the import system re-run the real module's own spec
        return importlib.util.spec_from_loader(fullname, loader=_Loader(module))


class _Loader:
    def __init__(self, module):
        self.module = module

    def create_module(self, spec):
        return self.module

    def exec_module(self, module):
        pass


import importlib.util  # noqa: E402

sys.meta_path.insert(0, _AliasFinder())
