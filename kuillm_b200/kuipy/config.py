"""Runtime switches of the kuipy front end.

The environment variable names and the module-level globals are those of the reference's
``kuipy/config.py`` (``KUIPY_JIT_STRICTNESS`` at config.py:43-46, ``KUIPY_JIT_VERBOSITY`` :38,
``KUIPY_PRINT_PROFILING`` :41, ``KUIPY_RE_TUNE`` :50, ``KUIPY_CACHE`` :24), because callers and
tests assign them directly (``kuipy.config.JIT_STRICTNESS = 2``).  Everything that configured
the F*/karamel/nvcc JIT pipeline is gone: kernels are compiled ahead of time into
``libkuiops.so``.
"""
import os
from pathlib import Path

_HERE = Path(__file__).resolve().parent
_PKG_ROOT = _HERE.parent


def _flag(name: str, default: str = "0") -> bool:
    return os.environ.get(name, default) == "1"


# Where tuned per-shape parameters are persisted (``tune_params`` JSON); the reference keeps
# its JIT cache under the same variable.
KUIPY_CACHE = Path(os.environ.get("KUIPY_CACHE", _PKG_ROOT / ".kuipy_cache")).resolve()
TUNE_FILE = KUIPY_CACHE / "tune_params.json"

# 0 = swallow kernel errors and fall back to PyTorch (one warning);
# 1 = raise when a selected kernel fails; 2 = also raise when an op is not offloaded.
JIT_STRICTNESS = int(os.environ.get("KUIPY_JIT_STRICTNESS", "1"))
# 1 = log kernel binding; 2 = also report every op that did not match
JIT_VERBOSITY = int(os.environ.get("KUIPY_JIT_VERBOSITY", "0"))
# record (op, argument signature) of every GPU-launching op instead of offloading
ENABLE_PRINT_PROFILING = _flag("KUIPY_PRINT_PROFILING")
# re-run the per-family tuners and write TUNE_FILE
RE_TUNE = _flag("KUIPY_RE_TUNE")
# accepted for compatibility; they steered the JIT toolchain and have no effect here
JIT_FULL_VERIFY = _flag("KUIPY_JIT_VERIFY")
JIT_FLUSH_CACHE = _flag("KUIPY_JIT_FLUSH_CACHE")
JIT_NVCC_FAST = _flag("KUIPY_JIT_NVCC_FAST")

# Which inputs ``supported()`` accepts:
#   "reference" - exactly the acceptance set of the reference gates (tile divisibility for
#                 mm/addmm, binary cat, full 2-D addmm bias, index shape <= input shape on every
#                 axis for gather ...), so its tests read the same;
#   "wide"      - everything the sm_100a kernels can take (any GEMM shape incl. M <= 16, 1-D
#                 bias, n-ary cat, causal/GQA attention, topk/isin/index/reduce families).
GATES = os.environ.get("KUIPY_GATES", "wide")


def reference_gates() -> bool:
    return GATES == "reference"


def nvcc_arch_flag() -> str:
    """The one architecture this library is built for."""
    return "-gencode=arch=compute_100a,code=sm_100a"


def ensure_dirs() -> None:
    KUIPY_CACHE.mkdir(parents=True, exist_ok=True)


def log(*parts) -> None:
    if JIT_VERBOSITY > 0:
        print("[kuipy]", *parts, flush=True)
