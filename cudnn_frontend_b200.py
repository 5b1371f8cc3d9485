"""Import shim: makes the package directory ``cudnn-frontend_b200/`` importable as
``cudnn_frontend_b200`` (a hyphen is not valid in a Python module name)."""

import importlib.util
import os
import sys

_pkg_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cudnn-frontend_b200")
_spec = importlib.util.spec_from_file_location(
    "cudnn_frontend_b200",
    os.path.join(_pkg_dir, "__init__.py"),
    submodule_search_locations=[_pkg_dir],
)
_module = importlib.util.module_from_spec(_spec)
sys.modules["cudnn_frontend_b200"] = _module
_spec.loader.exec_module(_module)
