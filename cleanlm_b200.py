"""Import shim: makes the package directory `clean-lm_b200/` importable as `cleanlm_b200`.

The directory name carries a hyphen, which the import statement cannot spell, so this module
loads it by path and replaces itself in `sys.modules` with the real package.
"""
import importlib.util
import pathlib
import sys

_dir = pathlib.Path(__file__).resolve().parent / "clean-lm_b200"
_spec = importlib.util.spec_from_file_location(
    __name__, _dir / "__init__.py", submodule_search_locations=[str(_dir)]
)
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
