"""Loader: makes the package directory `catena-lang_b200/` importable as `catena_lang_b200`
(a hyphen cannot appear in a Python module name)."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "catena-lang_b200")
_spec = importlib.util.spec_from_file_location(
    "catena_lang_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["catena_lang_b200"] = _mod
_spec.loader.exec_module(_mod)
