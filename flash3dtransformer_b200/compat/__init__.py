"""Run the reference's own host code (the `flash3dxfmr` Python package) on this library.

`install(reference_root)` makes `import flash3dxfmr` load the reference's unmodified Python files from
`<reference_root>/flash3dxfmr` with `compat/flash3dxfmr/lib/pshattn.py` standing where the reference's build would
install its compiled extension (CMakeLists.txt:69-76).  With `transformer_engine=True` the small stand-in package
beside this file is registered as `transformer_engine` when the real one is not importable (the reference's layers take
`Linear`, `LayerNorm` and `LayerNormMLP` from it: layers/psh_ops.py:13, layers/flash3d.py:12, layers/elem_wise.py:13).
A permanent installation needs no code from here: copy `compat/flash3dxfmr/lib/` into the reference checkout.
"""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))


def uninstall() -> None:
    """Forget every module `install` registered (the reference package and, if it was ours, transformer_engine)."""
    for name in list(sys.modules):
        mod = sys.modules[name]
        if name == "flash3dxfmr" or name.startswith("flash3dxfmr."):
            del sys.modules[name]
        elif (name == "transformer_engine" or name.startswith("transformer_engine.")) and \
                getattr(mod, "__file__", "") and os.path.abspath(mod.__file__).startswith(_HERE):
            del sys.modules[name]


def install(reference_root: str, transformer_engine: bool = True):
    """Import the reference's `flash3dxfmr` package from `reference_root` over this library and return it."""
    pkg_dir = os.path.join(reference_root, "flash3dxfmr")
    init = os.path.join(pkg_dir, "__init__.py")
    if not os.path.isfile(init):
        raise FileNotFoundError(f"{pkg_dir} is not the reference's Python package")
    uninstall()
    if transformer_engine:
        try:
            real = importlib.util.find_spec("transformer_engine")
        except (ImportError, ValueError):
            real = None
        if real is None:
            spec = importlib.util.spec_from_file_location(
                "transformer_engine", os.path.join(_HERE, "transformer_engine", "__init__.py"),
                submodule_search_locations=[os.path.join(_HERE, "transformer_engine")])
            te = importlib.util.module_from_spec(spec)
            sys.modules["transformer_engine"] = te
            spec.loader.exec_module(te)
    # the reference's files first, the folder holding lib/pshattn.py second: `..lib` resolves to the shim
    spec = importlib.util.spec_from_file_location(
        "flash3dxfmr", init, submodule_search_locations=[pkg_dir, os.path.join(_HERE, "flash3dxfmr")])
    pkg = importlib.util.module_from_spec(spec)
    sys.modules["flash3dxfmr"] = pkg
    try:
        spec.loader.exec_module(pkg)
    except Exception:
        uninstall()
        raise
    return pkg
