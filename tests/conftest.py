import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
# `import kuipy` resolves to the drop-in package; `oracle` and the golden helpers are test-only
for p in (ROOT / "kuillm_b200", ROOT, ROOT / "tests" / "golden"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture
def gates():
    """Switch the acceptance set for one test and restore it afterwards."""
    import kuipy.config as C
    from kuipy import registry
    saved = C.GATES

    def set_mode(mode):
        C.GATES = mode
        registry.reset()
    yield set_mode
    C.GATES = saved
    registry.reset()


@pytest.fixture
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("CUDA not available")
    return torch.device("cuda")
