"""Import shim: makes the package directory `lingbot-map_b200/` (a hyphen is not a legal module
name) importable as `lingbot_map_b200` whenever the repository root is on sys.path."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lingbot-map_b200")
_spec = importlib.util.spec_from_file_location(
    "lingbot_map_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["lingbot_map_b200"] = _mod
_spec.loader.exec_module(_mod)
