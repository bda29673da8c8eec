"""aten overload -> op family table and the dispatch entry point.

``try_dispatch(func, args, kwargs)`` returns the kernel's result, or ``None`` when no family
takes the call so that the caller falls through to stock PyTorch - the contract of the
reference's ``kuipy/registry.py:67-84``.  The table is built on first use from the overloads
each family declares.  Under ``config.GATES == "reference"`` it holds exactly the reference's
29 keys (its SDPA family exists but is left unconnected, registry.py:27-28,59 there); "wide"
gates add attention, the topk / isin / index / reduce families and the per-token data-movement
ops (casts, clone, masked_fill, argmax, embedding) the reference only lists as backlog.  Tuned parameters are loaded from and saved to ``config.TUNE_FILE``.
"""
import json

from . import config as C
from . import kuiops as K

_REGISTRY = None
_FAMILIES = None

_REFERENCE_FAMILIES = (K.ElementwiseImpl, K.MmImpl, K.BmmImpl, K.AddmmImpl, K.SoftmaxImpl,
                       K.GatherImpl, K.ScatterImpl, K.CatImpl, K.MeanImpl)
_WIDE_FAMILIES = (K.SdpaImpl, K.TopkImpl, K.IsinImpl, K.IndexImpl, K.ReduceImpl, K.DataMoveImpl)


def _load_tune_params():
    try:
        with open(C.TUNE_FILE) as f:
            data = json.load(f)
        return data if isinstance(data, dict) else {}
    except (OSError, ValueError):
        return {}


def _save_tune_params(params):
    C.ensure_dirs()
    with open(C.TUNE_FILE, "w") as f:
        json.dump(params, f, indent=1, sort_keys=True, default=list)


def _build_registry(tune_params):
    """One instance per family; every overload a family declares maps to that instance."""
    global _FAMILIES
    classes = _REFERENCE_FAMILIES if C.reference_gates() else _REFERENCE_FAMILIES + _WIDE_FAMILIES
    _FAMILIES = [cls(tune_params) for cls in classes]
    table = {}
    for fam in _FAMILIES:
        for overload in fam.overloads:
            table[overload] = fam
    return table


def _tune_impls(tune_params):
    for fam in _FAMILIES:
        tune_params = fam.tune(tune_params)
    return tune_params


def reset():
    """Drop the table so the next dispatch rebuilds it (after changing ``config.GATES``)."""
    global _REGISTRY, _FAMILIES
    _REGISTRY = None
    _FAMILIES = None


def table():
    global _REGISTRY
    if _REGISTRY is None:
        params = _load_tune_params()
        _REGISTRY = _build_registry(params)
        if C.RE_TUNE:
            _save_tune_params(_tune_impls(params))
    return _REGISTRY


def try_dispatch(func, args, kwargs):
    """Result of the kuiops kernel for ``func(*args, **kwargs)``, or None if nothing takes it."""
    fam = table().get(func)
    if fam is None:
        return None
    spec = fam.supported(func, args, kwargs)
    if spec is None:
        return None
    return fam.run(spec, args, kwargs)
