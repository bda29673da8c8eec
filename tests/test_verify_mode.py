"""Verify-mode bookkeeping (CPU only): the comparator and report that ``KuiperMode(verify=True)``
feeds.  Same behaviour the reference pins in its tests/test_verify_mode.py, including the cases it
keeps skipped while its attention family is disconnected."""
import io

import torch

import kuipy


class _Op:
    """Stand-in for an aten overload: only ``str()`` is used, as the statistics key."""
    def __init__(self, name):
        self._name = name

    def __str__(self):
        return self._name


def setup_function(_):
    kuipy.reset_verify()


def test_equal_tensors_pass():
    a = torch.randn(8, 8)
    kuipy._verify_compare(_Op("aten.mm"), a, a.clone(), tol=2e-2)
    s = kuipy.verify_stats["aten.mm"]
    assert (s["n"], s["fail"]) == (1, 0) and s["max_rel"] < 1e-6


def test_divergence_is_counted_and_described():
    a = torch.randn(8, 8)
    kuipy._verify_compare(_Op("aten.mm"), a, a + 0.5 * a.abs().mean(), tol=2e-2)
    s = kuipy.verify_stats["aten.mm"]
    assert s["fail"] == 1 and s["max_rel"] > 2e-2 and "rel=" in s["worst"]


def test_empty_reference_is_skipped():
    kuipy._verify_compare(_Op("aten.sdpa"), torch.randn(2, 3, 1), torch.randn(2, 3, 0), tol=2e-2)
    s = kuipy.verify_stats["aten.sdpa"]
    assert (s["n"], s["fail"]) == (0, 0)


def test_nonfinite_positions_are_ignored():
    out = torch.randn(4, 8)
    ref = out.clone()
    out[0], ref[0] = float("nan"), 0.0
    kuipy._verify_compare(_Op("aten.sdpa"), out, ref, tol=2e-2)
    s = kuipy.verify_stats["aten.sdpa"]
    assert (s["n"], s["fail"]) == (1, 0)


def test_tuple_outputs_are_paired():
    a, b = torch.randn(4, 4), torch.randn(4)
    kuipy._verify_compare(_Op("aten.sdpa"), (a, b, torch.zeros(2, dtype=torch.int64)),
                          (a.clone(), b.clone(), torch.ones(2, dtype=torch.int64)), tol=2e-2)
    assert kuipy.verify_stats["aten.sdpa"]["n"] == 2      # integer tensors are not compared


def test_shape_mismatch_fails():
    kuipy._verify_compare(_Op("aten.cat"), torch.randn(4, 4), torch.randn(4, 5), tol=2e-2)
    s = kuipy.verify_stats["aten.cat"]
    assert s["fail"] == 1 and "shape mismatch" in s["worst"]


def test_report_verdicts():
    buf = io.StringIO()
    assert kuipy.print_verify_report(out_dev=buf) is None and "no Kuiper-dispatched ops" in buf.getvalue()
    a = torch.randn(8, 8)
    kuipy._verify_compare(_Op("aten.mm"), a, a.clone(), tol=2e-2)
    buf = io.StringIO()
    assert kuipy.print_verify_report(out_dev=buf, tol=2e-2) is True and "PASS" in buf.getvalue()
    kuipy._verify_compare(_Op("aten.bmm"), a, a + 1.0, tol=2e-2)
    buf = io.StringIO()
    assert kuipy.print_verify_report(out_dev=buf, tol=2e-2) is False
    text = buf.getvalue()
    assert "FAIL (1 divergences)" in text and "[FAIL] aten.bmm" in text and "[ok  ] aten.mm" in text


def test_dispatch_falls_through_for_cpu_tensors_and_strictness_two_raises():
    import pytest
    import kuipy.config as C
    a, b = torch.randn(4, 4), torch.randn(4, 4)
    saved = C.JIT_STRICTNESS
    try:
        C.JIT_STRICTNESS = 1
        assert kuipy._jit_try(torch.ops.aten.mm.default, (a, b), {}) is None
        with kuipy.KuiperMode():
            assert torch.equal(torch.mm(a, b), a @ b)       # nothing offloaded, stock result
        C.JIT_STRICTNESS = 2
        with pytest.raises(RuntimeError):
            kuipy._jit_try(torch.ops.aten.mm.default, (a, b), {})
    finally:
        C.JIT_STRICTNESS = saved


def test_profile_signatures():
    sig = kuipy.print_call_data((torch.zeros(2, 3), [torch.zeros(1), 2], 1.5), {"dim": 0})
    assert "Tensor(nshape=2" in sig and "float" in sig and "dim=int" in sig
