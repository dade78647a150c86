"""Import shim: makes the package directory ``self-forcing_b200/`` importable as
``self_forcing_b200`` (a hyphen cannot appear in a Python module name)."""
import importlib.util
import pathlib
import sys

_dir = pathlib.Path(__file__).resolve().parent / "self-forcing_b200"
_spec = importlib.util.spec_from_file_location(
    __name__, _dir / "__init__.py", submodule_search_locations=[str(_dir)])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
