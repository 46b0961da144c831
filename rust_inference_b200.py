"""Import shim: makes the folder ``rust-inference_b200/`` importable as ``rust_inference_b200``.

The package folder carries the project's name, which has a hyphen and so cannot
be written in an ``import`` statement.  This file sits beside that folder; the
first ``import rust_inference_b200`` finds this file, loads the folder as a
regular package under the same module name and steps aside.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rust-inference_b200")
_spec = importlib.util.spec_from_file_location(
    "rust_inference_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir]
)
_mod = importlib.util.module_from_spec(_spec)
sys.modules["rust_inference_b200"] = _mod
_spec.loader.exec_module(_mod)
