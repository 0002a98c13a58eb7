"""Import shim: ``import llama_cl_b200`` loads the package in ``llama.cl_b200/``.

The package directory carries the reference project's name, which has a dot
in it and therefore cannot be spelled in an ``import`` statement.  This module
loads that directory under the importable name ``llama_cl_b200`` and replaces
itself with it in ``sys.modules``.
"""
import importlib.util as _ilu
import os as _os
import sys as _sys

_pkg_dir = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "llama.cl_b200")
_spec = _ilu.spec_from_file_location(
    "llama_cl_b200", _os.path.join(_pkg_dir, "__init__.py"), submodule_search_locations=[_pkg_dir])
_mod = _ilu.module_from_spec(_spec)
_sys.modules["llama_cl_b200"] = _mod
_spec.loader.exec_module(_mod)
