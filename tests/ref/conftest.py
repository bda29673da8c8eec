"""Runs the reference project's own test files, unmodified, against the drop-in ``kuipy``.

The files are not part of this repository.  ``stage_reference_tests()`` (called by the build
entry point wherever a checkout of the reference is present) copies them byte for byte into
``_staged/`` next to this file, which version control ignores; only the file name gets a
``test_ref_`` prefix so that it does not collide with this repository's own tests of the same
name.  When nothing is staged the directory simply collects no tests.

Every staged test is marked ``gpu`` and runs under the reference's acceptance set
(``config.GATES = "reference"``): the reference tests assert rejections (three-tensor cat,
broadcast addmm bias, K = 63 ...) that only that set reproduces.  Module-level switches the
tests assign (``kuipy.config.JIT_STRICTNESS = 2``) are restored after each test.
"""
import hashlib
import os
import shutil
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent
STAGED = HERE / "_staged"
REFERENCE_TESTS = Path(os.environ.get("KUILLM_REFERENCE", "/root/reference")) / "tests"
FILES = ("test_jit_ops.py", "test_jit_general.py", "test_verify_mode.py")


def stage_reference_tests() -> int:
    """Copy the reference's test files into ``_staged/``; returns how many are now staged."""
    if not REFERENCE_TESTS.is_dir():
        return len(list(STAGED.glob("test_ref_*.py"))) if STAGED.is_dir() else 0
    STAGED.mkdir(exist_ok=True)
    n = 0
    manifest = []
    for name in FILES:
        src = REFERENCE_TESTS / name
        if not src.is_file():
            continue
        dst = STAGED / ("test_ref_" + name[len("test_"):])
        shutil.copyfile(src, dst)
        manifest.append(f"{hashlib.sha256(dst.read_bytes()).hexdigest()}  {dst.name}  <- tests/{name}")
        n += 1
    (STAGED / "MANIFEST.txt").write_text("\n".join(manifest) + "\n")
    return n


def pytest_collection_modifyitems(config, items):
    for item in items:
        if STAGED in Path(str(item.fspath)).parents:
            item.add_marker(pytest.mark.gpu)


@pytest.fixture(autouse=True)
def _reference_acceptance_set(request):
    if STAGED not in Path(str(request.node.fspath)).parents:
        yield
        return
    import kuipy.config as C
    from kuipy import registry
    saved = (C.GATES, C.JIT_STRICTNESS, C.JIT_VERBOSITY)
    C.GATES = "reference"
    registry.reset()
    yield
    C.GATES, C.JIT_STRICTNESS, C.JIT_VERBOSITY = saved
    registry.reset()
