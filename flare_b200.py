"""Import shim: makes the package directory ``flare.py_b200/`` importable as ``flare_b200``.

A directory name with a dot in it cannot be imported by the normal machinery,
so this module loads ``flare.py_b200/__init__.py`` as a package and replaces
itself with it in ``sys.modules``.
"""
import importlib.util
import sys
from pathlib import Path

_pkg_dir = Path(__file__).resolve().parent / "flare.py_b200"
_spec = importlib.util.spec_from_file_location(
    "flare_b200", _pkg_dir / "__init__.py", submodule_search_locations=[str(_pkg_dir)])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["flare_b200"] = _mod
_spec.loader.exec_module(_mod)
