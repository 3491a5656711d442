"""Import name for the package whose sources live in ``kir-ai_b200/``.

A hyphen cannot appear in a Python module name, so ``import kirai_b200`` finds
this file, which loads ``kir-ai_b200/__init__.py`` as the package
``kirai_b200`` (sub-packages resolve inside that folder) and puts it in
``sys.modules`` in place of itself.
"""
import importlib.util
import pathlib
import sys

_dir = pathlib.Path(__file__).resolve().parent / "kir-ai_b200"
_spec = importlib.util.spec_from_file_location(
    "kirai_b200", _dir / "__init__.py", submodule_search_locations=[str(_dir)]
)
_module = importlib.util.module_from_spec(_spec)
sys.modules["kirai_b200"] = _module
_spec.loader.exec_module(_module)
