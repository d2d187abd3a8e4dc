"""Packaging entry point.  ``pip install .`` (or ``python setup.py build_ext --inplace``) compiles the native
extension with nvcc for sm_100a through ``deepep_b200._build`` (the same in-tree build the tests use) and ships
``deepep_b200/_C*.so`` together with ``_build_info.json``; the sources travel along so the extension can be rebuilt.

Parity: ``setup.py:42-44`` / ``build_support.py:280-430`` of the reference (one build hook that compiles the device
code and records the build provenance).
"""
import importlib.util
import os
import sys

from setuptools import Extension, setup
from setuptools.command.build_ext import build_ext

ROOT = os.path.dirname(os.path.abspath(__file__))


def _load_build_module():
    spec = importlib.util.spec_from_file_location("deepep_b200_build", os.path.join(ROOT, "deepep_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class NvccBuild(build_ext):
    """Delegates to deepep_b200/_build.py and copies the product next to the Python sources of the build tree."""

    def run(self):
        builder = _load_build_module()
        product = builder.build(verbose=bool(os.environ.get("DEEPEP_BUILD_VERBOSE")))
        if not self.inplace:
            target_dir = os.path.join(self.build_lib, "deepep_b200")
            os.makedirs(target_dir, exist_ok=True)
            self.copy_file(str(product), os.path.join(target_dir, os.path.basename(str(product))))
            info = os.path.join(ROOT, "deepep_b200", "_build_info.json")
            if os.path.exists(info):
                self.copy_file(info, os.path.join(target_dir, "_build_info.json"))


if __name__ == "__main__":
    sys.path.insert(0, ROOT)
    setup(ext_modules=[Extension("deepep_b200._C", sources=[])], cmdclass={"build_ext": NvccBuild})
