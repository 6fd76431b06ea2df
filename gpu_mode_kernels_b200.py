"""Importable alias of the package directory ``gpu-mode-kernels_b200/``.

A hyphen is not valid in a Python module name, so ``import gpu_mode_kernels_b200``
loads the package that lives in the hyphenated directory beside this file and
installs it in ``sys.modules`` under this name (sub-modules resolve normally).
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gpu-mode-kernels_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir]
)
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
