"""Helpers shared by the GPU parity tests: tensor <-> numpy, and the three parity bars."""
import numpy as np
import torch

from oracle import kuiops_oracle as O


def to_np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.float()
    return t.numpy()


def run_family(impl, func, args, kwargs=None):
    """What the reference tests do: ask the gate, then run the kernel behind it."""
    kwargs = kwargs or {}
    spec = impl.supported(func, args, kwargs)
    assert spec is not None, "expected a supported spec"
    return impl.run(spec, args, kwargs)


def assert_close_ref_bar(out, ref_np, dtype):
    """Both bars at once.  The reference's own (tests/test_jit_ops.py:34-43 there): fp32
    allclose(1e-3, 1e-3); bf16 / fp16 relative Frobenius norm < 3e-2.  And, for bf16 / fp16, the
    stricter element-wise one: max |out - ref| / max |ref| <= 2e-2 against the fp64 oracle, so that
    a wrong edge element of a ragged shape cannot hide under a norm."""
    o = to_np(out).astype(np.float64)
    assert o.shape == ref_np.shape, (o.shape, ref_np.shape)
    if dtype == torch.float32:
        np.testing.assert_allclose(o, ref_np, atol=1e-3, rtol=1e-3)
    else:
        rel = O.rel_frobenius(o, ref_np)
        assert rel < 3e-2, f"relative norm {rel:.4f} too large"
        err = O.max_rel_err(o, ref_np)
        assert err <= 2e-2, f"max relative error {err:.3e} > 2e-2"


def assert_max_rel(out, ref_np, tol=2e-2):
    """bf16 GEMM / attention bar: max |out - ref| / max |ref| <= tol against an fp64 reference."""
    err = O.max_rel_err(to_np(out), ref_np)
    assert err <= tol, f"max relative error {err:.3e} > {tol:.1e}"


def assert_fp32_1e5(out, ref_np):
    """fp32 softmax / mean / reduce bar: within 1e-5 (relative, with a matching absolute floor)."""
    np.testing.assert_allclose(to_np(out).astype(np.float64), ref_np, rtol=1e-5, atol=1e-5 * float(np.abs(ref_np).max()))


def assert_bit_exact(out, ref_np):
    o = to_np(out)
    assert o.shape == ref_np.shape and o.dtype == ref_np.dtype, (o.shape, o.dtype, ref_np.shape, ref_np.dtype)
    assert np.array_equal(o, ref_np)
