"""kuillm_b200: a B200 (sm_100a) implementation of the kuiops operator library.

``kuillm_b200.kuipy`` is the drop-in ``kuipy`` package (dispatch mode, op table, op families);
``kuillm_b200/csrc`` holds the CUDA kernels and the C ABI declared in ``include/kuiops.h``;
``kuillm_b200/lib/libkuiops.so`` is the built library.  Put this directory on ``sys.path`` (or
call ``install_as_kuipy()``) and ``import kuipy`` resolves to the package here.
"""
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent


def install_as_kuipy():
    """Make ``import kuipy`` resolve to ``kuillm_b200.kuipy`` in this process."""
    p = str(PACKAGE_DIR)
    if p not in sys.path:
        sys.path.insert(0, p)
    import kuipy  # noqa: F401
    return sys.modules["kuipy"]


def build(force=False, verbose=False):
    """Compile ``libkuiops.so`` for sm_100a."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("kuiops_build", PACKAGE_DIR / "csrc" / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(force=force, verbose=verbose)
