"""Handle cache and dispatch-mode integration on a GPU (the reference's tests/test_jit_general.py)."""
import time

import pytest
import torch

import kuipy
import kuipy.config
from kuipy import compile as jit_compile
from kuipy import kuiops
from _util import run_family

pytestmark = pytest.mark.gpu
aten = torch.ops.aten


@pytest.fixture(autouse=True)
def _strictness():
    saved = kuipy.config.JIT_STRICTNESS
    yield
    kuipy.config.JIT_STRICTNESS = saved


def test_cache_is_hot_on_second_call(cuda):
    kuipy.config.JIT_STRICTNESS = 2
    impl = kuiops.MmImpl({})
    A, B = torch.randn(64, 64, device="cuda"), torch.randn(64, 64, device="cuda")
    run_family(impl, aten.mm.default, (A, B))
    before = set(jit_compile._loaded.keys())
    assert before, "the first call must register a kernel handle"
    t0 = time.time()
    run_family(impl, aten.mm.default, (A, B))
    assert set(jit_compile._loaded.keys()) == before
    assert time.time() - t0 < 2.0


def test_kuiper_mode_integration(cuda):
    kuipy.config.JIT_STRICTNESS = 2
    A, B = torch.randn(128, 64, device="cuda"), torch.randn(64, 128, device="cuda")
    with kuipy.KuiperMode():
        out = torch.mm(A, B)
    assert torch.allclose(out, A @ B, atol=1e-3, rtol=1e-3)


def test_unsupported_falls_through(cuda, gates):
    gates("reference")
    impl = kuiops.MmImpl({})
    # K = 63 divides no block-K tile of the reference kernels
    assert impl.supported(aten.mm.default, (torch.randn(128, 63, device="cuda"), torch.randn(63, 128, device="cuda")), {}) is None
    assert impl.supported(aten.mm.default, (torch.randn(64, 64), torch.randn(64, 64)), {}) is None
    gates("wide")
    assert impl.supported(aten.mm.default, (torch.randn(128, 63, device="cuda"), torch.randn(63, 128, device="cuda")), {}) is not None
    assert impl.supported(aten.mm.default, (torch.randn(64, 64), torch.randn(64, 64)), {}) is None


def test_verify_mode_counts_offloaded_ops(cuda, gates):
    gates("wide")
    kuipy.config.JIT_STRICTNESS = 1
    kuipy.reset_verify()
    A, B = torch.randn(64, 64, device="cuda", dtype=torch.bfloat16), torch.randn(64, 64, device="cuda", dtype=torch.bfloat16)
    with kuipy.KuiperMode(verify=True, verify_tol=2e-2):
        torch.mm(A, B)
        torch.softmax(A.float(), -1)
        torch.cat([A, B], 0)
    assert kuipy.verify_stats["aten.mm.default"]["n"] == 1
    assert kuipy.verify_stats["aten._softmax.default"]["fail"] == 0
    import io
    buf = io.StringIO()
    assert kuipy.print_verify_report(out_dev=buf) is True


def test_sampling_path_under_dispatch_mode(cuda, gates):
    """softmax -> topk -> gather / isin / cat as a sampler issues them, all offloaded."""
    gates("wide")
    kuipy.config.JIT_STRICTNESS = 1
    g = torch.Generator().manual_seed(0)
    logits = (torch.randn(8, 5000, generator=g) * 3).cuda()
    stop = torch.randint(0, 5000, (64,), generator=g).cuda()
    from kuipy import _ffi
    n0 = _ffi.launch_count()
    with kuipy.KuiperMode():
        p = torch.softmax(logits, -1)
        v, i = torch.topk(p, 50)
        picked = torch.gather(i, 1, torch.zeros(8, 1, dtype=torch.int64, device="cuda"))
        done = torch.isin(picked, stop)
        seq = torch.cat([picked, picked, picked], 1)
    assert _ffi.launch_count() - n0 >= 5
    rp = torch.softmax(logits, -1)
    assert torch.allclose(p, rp, rtol=1e-5, atol=1e-9)
    assert torch.equal(i[:, 0], rp.argmax(-1)) and seq.shape == (8, 3) and done.dtype == torch.bool
