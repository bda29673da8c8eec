"""Kernel handles for the op families.

In the reference this module renders an F* instantiation, extracts CUDA through karamel and
builds one torch extension per instantiation (kuipy/compile.py:86-130), memoising the loaded
module in ``_loaded`` and build failures in ``_failed`` (:21-25).  Here every kernel is already
inside ``libkuiops.so``; ``build_kernel`` keeps its signature and its two caches, but a "build"
is a lookup of the family's binder followed by closing it over the instantiation parameters.
The returned handle has the ``run(...)`` entry of the matching wrapper template.
"""
from . import _ffi
from . import config as C

# ext_name -> handle.  Same keying as the reference: module name with dots replaced.
_loaded = {}
# ext_name -> exception raised while binding; re-raised on every later request.
_failed = {}

# wrapper template name -> callable(ctx) -> handle; filled by kuipy.kuiops at import
_binders = {}


class KernelHandle:
    """What ``build_kernel`` returns: an object with ``run``, like a loaded extension module."""
    __slots__ = ("name", "run")

    def __init__(self, name, run):
        self.name = name
        self.run = run

    def __repr__(self):
        return f"<kuiops kernel {self.name}>"


def register_binder(wrapper_template, binder):
    _binders[wrapper_template] = binder


def build_kernel(module: str, fst_template: str, fst_ctx: dict, wrapper_template: str, wrapper_ctx: dict):
    """Return the handle for instantiation ``module`` of the family behind ``wrapper_template``.

    ``fst_template`` / ``fst_ctx`` named the F* instantiation in the reference; they are kept
    in the signature and only ``fst_ctx`` is consulted, for parameters the wrapper context lacks.
    """
    ext_name = module.replace(".", "_")
    hit = _loaded.get(ext_name)
    if hit is not None:
        return hit
    err = _failed.get(ext_name)
    if err is not None:
        raise err
    try:
        _ffi.lib()                                  # fails loudly when the CUDA library is absent
        binder = _binders.get(wrapper_template)
        if binder is None:
            raise KeyError(f"no kuiops kernel family is bound to {wrapper_template!r}")
        ctx = dict(fst_ctx)
        ctx.update(wrapper_ctx)
        handle = KernelHandle(ext_name, binder(ctx))
        C.log(f"bound {ext_name}")
    except Exception as e:  # negative cache, as the reference does for failed builds
        _failed[ext_name] = e
        raise
    _loaded[ext_name] = handle
    return handle
