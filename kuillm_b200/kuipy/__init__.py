"""kuipy: route eligible aten calls to the kuiops sm_100a kernels.

Drop-in for the reference package of the same name: ``KuiperMode`` (a ``TorchDispatchMode``,
kuipy/__init__.py:133-178 there), ``is_available``, the verify-mode comparator and report
(:193-245) and the print-profiling collector (:252-263) keep their names, arguments and
printed text.  ``is_available()`` used to mean "the F* toolchain is installed"; it now means
"libkuiops.so loads and a CUDA device is present".
"""
import sys

from . import config as C

__all__ = ["KuiperMode", "is_available", "reset_verify", "verify_stats", "print_verify_report",
           "print_profile_data", "config", "registry", "kuiops", "compile"]


def is_available() -> bool:
    try:
        import torch
        if not torch.cuda.is_available():
            return False
        from . import _ffi
        return _ffi.is_loadable()
    except Exception:
        return False


# ---------------------------------------------------------------------------------------------
# call signatures for the print-profiling mode
# ---------------------------------------------------------------------------------------------
_LIST_MARK = 0x67


def arg_data(a):
    """Hashable summary of one argument: tensors by (rank or shape, dtype, device)."""
    import torch
    if isinstance(a, torch.Tensor):
        return (tuple(a.shape) if C.JIT_VERBOSITY > 1 else a.dim(), a.dtype, a.device)
    if isinstance(a, (list, tuple)):
        return (_LIST_MARK, tuple(arg_data(x) for x in a))
    if isinstance(a, (torch.dtype, torch.device, bool)):
        return a
    return type(a).__name__


def print_arg_data(a):
    try:
        if isinstance(a, tuple) and a and a[0] == _LIST_MARK:
            return "[" + ", ".join(print_arg_data(x) for x in a[1]) + ", ]"
        if isinstance(a, tuple) and len(a) == 3:
            shape, dtype, device = a
            return f"Tensor(nshape={shape}, dtype={dtype}, device={device})"
    except Exception:
        pass
    return str(a)


def print_call_data_aux(args, kwargs_keys, kwargs_values, ret):
    kw = ", ".join(f"{k}={print_arg_data(v)}" for k, v in zip(kwargs_keys, kwargs_values))
    return f"args={[print_arg_data(a) for a in args]}, kwargs={{ {kw} }} -> {print_arg_data(ret)}"


def print_call_data(args, kwargs):
    return print_call_data_aux(tuple(arg_data(a) for a in args), tuple(kwargs.keys()),
                               tuple(arg_data(v) for v in kwargs.values()), "no return captured")


# ---------------------------------------------------------------------------------------------
# dispatch with the strictness ladder
# ---------------------------------------------------------------------------------------------
_jit_dispatch = None
_jit_warned = False


def _jit_try(func, args, kwargs, VERY_STRICT=False):
    """Kernel result for the call, or None.  Strictness 0 swallows kernel errors (one warning)
    and returns None; >= 1 re-raises them; 2 also raises when the op was not offloaded."""
    global _jit_dispatch, _jit_warned
    if _jit_dispatch is None:
        from .registry import try_dispatch
        _jit_dispatch = try_dispatch
    try:
        out = _jit_dispatch(func, args, kwargs)
    except Exception as e:
        if C.JIT_STRICTNESS > 0:
            raise
        if not _jit_warned:
            _jit_warned = True
            print(f"[kuipy] JIT dispatch failed, falling back to PyTorch: {e}", file=sys.stderr)
        out = None
    if out is None:
        if C.JIT_VERBOSITY > 1:
            print(f"[kuipy] operator {func} ({print_call_data(args, kwargs)}) did not match", file=sys.stderr)
        if C.JIT_STRICTNESS > 1 or VERY_STRICT:
            raise RuntimeError(f"[kuipy] operator {func} was not offloaded (strictness {C.JIT_STRICTNESS})")
    return out


def _tensors(x):
    import torch
    if isinstance(x, torch.Tensor):
        yield x
    elif isinstance(x, (list, tuple)):
        for item in x:
            yield from _tensors(item)


def _launches_gpu_kernel(func, args, out):
    """False for pure view ops: every output aliases an input's storage and nothing is mutated."""
    if func._schema.is_mutable:
        return True
    inputs = {t.untyped_storage().data_ptr() for t in _tensors(args)}
    outputs = list(_tensors(out))
    return not (outputs and all(t.untyped_storage().data_ptr() in inputs for t in outputs))


def _has_cuda_kernel(func):
    import torch
    try:
        return torch._C._dispatch_has_kernel_for_dispatch_key(func.name(), torch._C.DispatchKey.CUDA)
    except Exception:
        return False


profile_data = set()
_mode_class = None


def _make_mode_class():
    global _mode_class
    if _mode_class is not None:
        return _mode_class
    from torch.utils._python_dispatch import TorchDispatchMode

    class KuiperMode(TorchDispatchMode):
        """``with kuipy.KuiperMode(): model(...)`` runs every eligible aten call on a kuiops
        kernel and everything else on stock PyTorch.  With ``verify=True`` each offloaded,
        non-mutating call is also run by PyTorch and the two results are compared (relative
        Frobenius norm against ``verify_tol``); see ``print_verify_report``."""
        dummy_print_mode = False   # profile only, never offload

        def __init__(self, verify=False, verify_tol=2e-2):
            super().__init__()
            self.verify = verify
            self.verify_tol = verify_tol

        def __torch_dispatch__(self, func, types, args=(), kwargs=None):
            kwargs = kwargs or {}
            out = None if self.dummy_print_mode else _jit_try(func, args, kwargs)
            if out is None:
                out = func(*args, **kwargs)
            elif self.verify and not func._schema.is_mutable:
                _verify_compare(func, out, func(*args, **kwargs), self.verify_tol)
            if C.ENABLE_PRINT_PROFILING and _launches_gpu_kernel(func, args, out):
                profile_data.add((func, tuple(arg_data(a) for a in args), tuple(kwargs.keys()),
                                  tuple(arg_data(v) for v in kwargs.values()), arg_data(out)))
            return out

    _mode_class = KuiperMode
    return KuiperMode


def __getattr__(name):
    # built lazily so that importing kuipy does not import torch
    if name == "KuiperMode":
        return _make_mode_class()
    if name in ("registry", "kuiops", "compile", "inductor"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)


# ---------------------------------------------------------------------------------------------
# verify mode: kuiops result against stock PyTorch
# ---------------------------------------------------------------------------------------------
verify_stats = {}     # str(func) -> {"n", "fail", "max_rel", "worst"}


def reset_verify():
    verify_stats.clear()


def _verify_compare(func, out, ref, tol):
    """Fold one comparison into ``verify_stats[str(func)]``.  Floating tensors are paired in
    order and compared by ||out - ref|| / ||ref|| over the positions where both are finite
    (fully masked attention rows are implementation-defined); empty tensors are skipped and a
    shape mismatch counts as a failure."""
    import torch
    entry = verify_stats.setdefault(str(func), {"n": 0, "fail": 0, "max_rel": 0.0, "worst": None})
    for o, r in zip(_tensors(out), _tensors(ref)):
        if not (o.is_floating_point() and r.is_floating_point()):
            continue
        if o.numel() == 0 or r.numel() == 0:
            continue
        if o.shape != r.shape:
            entry["fail"] += 1
            entry["worst"] = f"shape mismatch {tuple(o.shape)} vs {tuple(r.shape)}"
            continue
        o32, r32 = o.float(), r.float()
        ok = torch.isfinite(o32) & torch.isfinite(r32)
        if not ok.any():
            continue
        diff, base = (o32 - r32)[ok], r32[ok]
        rel = (diff.norm() / (base.norm() + 1e-12)).item()
        entry["n"] += 1
        entry["max_rel"] = max(entry["max_rel"], rel)
        if rel > tol:
            entry["fail"] += 1
            entry["worst"] = f"rel={rel:.3e} (tol {tol:.1e})"


def print_verify_report(out_dev=sys.stdout, tol=2e-2):
    """Per-op summary of a verify run; returns True when nothing diverged."""
    if not verify_stats:
        print("[verify] no Kuiper-dispatched ops were checked.", file=out_dev)
        return
    failures = sum(e["fail"] for e in verify_stats.values())
    print(f"[verify] Kuiper vs stock PyTorch (relative Frobenius norm, tol {tol:.1e}):", file=out_dev)
    for name in sorted(verify_stats):
        e = verify_stats[name]
        mark = "FAIL" if e["fail"] else "ok"
        line = f"  [{mark:4}] {name}: {e['n']} checked, {e['fail']} fail, max_rel={e['max_rel']:.3e}"
        if e["worst"]:
            line += f", worst: {e['worst']}"
        print(line, file=out_dev)
    print("[verify] result: " + ("PASS" if failures == 0 else f"FAIL ({failures} divergences)"), file=out_dev)
    return failures == 0


def print_profile_data(out_dev=sys.stdout):
    """Dump the call signatures collected under KUIPY_PRINT_PROFILING, grouped by op."""
    by_op = {}
    for func, args, kw_keys, kw_vals, ret in profile_data:
        by_op.setdefault(func, []).append(print_call_data_aux(args, kw_keys, kw_vals, ret))
    for func, calls in by_op.items():
        note = "" if _has_cuda_kernel(func) else "  [no CUDA kernel: composite — internal GPU sub-ops not interceptable]"
        print(f"Function {func}:{note}", file=out_dev)
        for c in calls:
            print(f"  {c}", file=out_dev)
