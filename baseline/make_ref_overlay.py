"""Assemble an importable copy of the reference's grouped-GEMM operators under baseline/_ref/.

The reference's hot-path kernels are Python (CuTe DSL) and only need the package skeleton around
them.  The pip-installed cudnn wheel of this image is an older release whose compiled module
lacks two names the reference's ``python/cudnn/__init__.py`` imports, so the overlay takes
``__init__.py``, ``graph.py``, ``wrapper.py`` and the compiled module from the installed wheel and
``api_base.py``, ``datatypes.py``, ``grouped_gemm/`` and ``discrete_grouped_gemm/`` from the
reference checkout.  baseline/_ref/ is not tracked by git; it exists so that the reference's own
kernels can be run next to this repository's on a GPU box.

    REFERENCE_ROOT=<reference checkout> python baseline/make_ref_overlay.py

Without REFERENCE_ROOT the checkout is looked for in a directory ``reference`` next to this
repository.
"""

import importlib.util
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
DST = os.path.join(HERE, "_ref", "cudnn")


def main():
    spec = importlib.util.find_spec("cudnn")
    if spec is None or not spec.submodule_search_locations:
        sys.exit("the cudnn wheel is not installed: cannot build the overlay")
    installed = list(spec.submodule_search_locations)[0]
    if os.path.exists(DST):
        shutil.rmtree(DST)
    os.makedirs(DST)
    for name in os.listdir(installed):
        if name in ("__init__.py", "graph.py", "wrapper.py") or name.startswith("_compiled_module"):
            shutil.copy2(os.path.join(installed, name), os.path.join(DST, name))
    src = os.path.join(REF, "python", "cudnn")
    for name in ("api_base.py", "datatypes.py"):
        shutil.copy2(os.path.join(src, name), os.path.join(DST, name))
    for name in ("grouped_gemm", "discrete_grouped_gemm"):
        shutil.copytree(os.path.join(src, name), os.path.join(DST, name), ignore=shutil.ignore_patterns("__pycache__"))
    print("overlay written to", DST)


if __name__ == "__main__":
    main()
