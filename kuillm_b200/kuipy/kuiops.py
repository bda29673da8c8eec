"""Op families: which aten calls the kuiops kernels take, and how they are launched.

Same contract as the reference's ``kuipy/kuiops.py``: every family object has
``supported(func, args, kwargs) -> spec | None`` (never raises for an ineligible call) and
``run(spec, args, kwargs) -> Tensor | tuple`` (raises when the kernel cannot be bound or
launched), plus the ``fst_template`` / ``wrapper_template`` / ``tune_key`` / ``tune_params``
class attributes and ``tune()`` (kuipy/kuiops.py:27-43 there).  ``run`` still goes through
``compile.build_kernel`` with a module name per instantiation, so the ``_loaded`` cache behaves
as before; the handle it gets back calls straight into ``libkuiops.so``.

Two acceptance sets exist (``config.GATES``).  "reference" answers exactly as the reference
gates do on the dtypes the sm_100a kernels implement (fp32 / bf16 / fp16 payloads); "wide"
also accepts what only the new kernels can do.  Deviation that holds in both: fp64 and unsigned
integer arithmetic maps are not offloaded (the reference lists them in ``_SCALAR_DTYPES``,
kuiops.py:106-111).
"""
import math

import torch

from . import _ffi
from . import compile as _compile
from . import config as C

aten = torch.ops.aten

# Kuiper's launch limits (max_blocks, max_blocks * max_threads): the reference gates sizes with
# them (kuiops.py:12,514).  The new kernels are grid-stride, so "wide" gates only use the first
# as a sanity bound on element counts.
_MAX_BLOCKS = 2097152
_MAX_NUMEL = _MAX_BLOCKS * 1024

_KERNEL_FLOATS = (torch.float32, torch.bfloat16, torch.float16)
_TAG = {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16", torch.float64: "f64",
        torch.int64: "i64", torch.int32: "i32", torch.int16: "i16", torch.int8: "i8",
        torch.uint8: "u8", torch.bool: "u8"}


def torch_dtype_to_fstar(dt):
    """Short element-type tag used in module names (the reference's F* type names)."""
    return _TAG[dt]


def _is_cuda_tensor(x):
    return isinstance(x, torch.Tensor) and x.is_cuda


def _scalar(x):
    """Python number, or a 0-d float64 tensor (how a Python float reaches aten), else None."""
    if isinstance(x, bool):
        return None
    if isinstance(x, (int, float)):
        return x
    if isinstance(x, torch.Tensor) and x.dim() == 0 and x.dtype == torch.float64:
        return float(x.item())
    return None


def _wrap_dim(d, rank):
    d = int(d)
    return d + rank if d < 0 else d


def _ints(shape):
    return [int(s) for s in shape]


def _prod(dims):
    n = 1
    for d in dims:
        n *= int(d)
    return n


def _pointwise_le(small, big):
    return len(small) == len(big) and all(a <= b for a, b in zip(small, big))


class _Family:
    fst_template = None
    wrapper_template = None
    tune_key = ""
    tune_params = ()

    def __init__(self, all_tune_params):
        self.tune_params = all_tune_params.get(self.tune_key, self.tune_params)

    def _mod(self, module, fst_ctx, wrapper_ctx):
        return _compile.build_kernel(module, self.fst_template, fst_ctx, self.wrapper_template, wrapper_ctx)

    def tune(self, all_tune_params):
        all_tune_params[self.tune_key] = self.tune_params
        return all_tune_params


# =============================================================================================
# elementwise maps
# =============================================================================================
def _const_tag(consts):
    if not consts:
        return ""
    out = []
    for c in consts:
        txt = repr(c).replace("-", "n").replace(".", "p").replace("+", "")
        out.append("".join(ch for ch in txt if ch.isalnum()))
    return "C" + "_".join(out)


class ElementwiseImpl(_Family):
    """21 aten overloads over same-shape operands, no broadcasting (kuiops.py:150-320 there)."""
    fst_template = "elementwise/Kuiops.Elementwise.Inst.fst.j2"
    wrapper_template = "elementwise/wrapper_elementwise.cu.j2"
    tune_key = "ELEM"
    tune_params = ()

    _ARITH = {
        aten.silu.default: "silu", aten.neg.default: "neg", aten.rsqrt.default: "rsqrt",
        aten.cos.default: "cos", aten.sin.default: "sin", aten.pow.Tensor_Scalar: "pow",
        aten.add.Tensor: "add", aten.add.Scalar: "add", aten.mul.Tensor: "mul", aten.mul.Scalar: "mul",
        aten.sub.Tensor: "sub", aten.sub.Scalar: "sub", aten.div.Tensor: "div", aten.div.Scalar: "div",
    }
    _COMPARE = {aten.eq.Scalar: "eq", aten.le.Scalar: "le", aten.lt.Scalar: "lt"}
    _BIT1 = {aten.bitwise_not.default: "bnot"}
    _BIT2 = {aten.bitwise_and.Tensor: "band", aten.bitwise_or.Tensor: "bor"}
    overloads = tuple(_ARITH) + tuple(_COMPARE) + tuple(_BIT1) + tuple(_BIT2) + (aten.where.self,)

    def supported(self, func, args, kwargs):
        if not args:
            return None
        A = args[0]
        if func is aten.where.self:
            return self._where_spec(args)
        if not (_is_cuda_tensor(A) and 0 < A.numel() <= _MAX_NUMEL):
            return None

        def same_as_A(B):
            return _is_cuda_tensor(B) and B.dtype == A.dtype and tuple(B.shape) == tuple(A.shape)

        if func in self._BIT1:
            if A.dtype != torch.bool:
                return None
            return dict(kind="map_u8", method=self._BIT1[func], dtype=A.dtype, consts=[], call=[A])
        if func in self._BIT2:
            if A.dtype != torch.bool or len(args) < 2 or not same_as_A(args[1]):
                return None
            return dict(kind="map_u8", method=self._BIT2[func], dtype=A.dtype, consts=[], call=[A, args[1]])
        if func in self._COMPARE:
            s = _scalar(args[1]) if len(args) > 1 else None
            if A.dtype not in _KERNEL_FLOATS or s is None:
                return None
            return dict(kind="map_nip", method=self._COMPARE[func], dtype=A.dtype, consts=[s], call=[A])
        method = self._ARITH.get(func)
        if method is None or A.dtype not in _KERNEL_FLOATS:
            return None
        if len(args) == 1:
            return dict(kind="map", method=method, dtype=A.dtype, consts=[], call=[A])
        alpha = 1
        if method in ("add", "sub") and kwargs.get("alpha", 1) != 1:
            alpha = _scalar(kwargs["alpha"])
            if alpha is None:
                return None
        if func is aten.pow.Tensor_Scalar and isinstance(args[1], int) and not isinstance(args[1], bool) and args[1] == 2:
            return dict(kind="map", method="square", dtype=A.dtype, consts=[], call=[A])
        s = _scalar(args[1])
        if s is not None:
            return dict(kind="map", method=method, dtype=A.dtype, consts=[s, alpha], call=[A])
        if same_as_A(args[1]):
            return dict(kind="map2", method=method, dtype=A.dtype, consts=[alpha], call=[A, args[1]])
        return None

    @staticmethod
    def _where_spec(args):
        if len(args) < 3:
            return None
        Cnd, X, Y = args[0], args[1], args[2]
        if not all(_is_cuda_tensor(t) for t in (Cnd, X, Y)):
            return None
        if Cnd.dtype not in (torch.bool, torch.uint8) or X.dtype != Y.dtype:
            return None
        if not (tuple(Cnd.shape) == tuple(X.shape) == tuple(Y.shape)):
            return None
        if not (0 < X.numel() <= _MAX_NUMEL) or X.element_size() not in (1, 2, 4, 8):
            return None
        return dict(kind="map3", method="bwhere", dtype=X.dtype, consts=[], call=[Cnd, X, Y])

    def run(self, spec, args, kwargs):
        kind, method, dt = spec["kind"], spec["method"], spec["dtype"]
        tag = _const_tag(spec["consts"])
        module = f"Kuiops.Elementwise.{kind.title().replace('_', '')}.{method.title()}.{_TAG[dt].title()}"
        if tag:
            module += f".{tag}"
        name = f"elem_{kind}_{method}_{_TAG[dt]}_{tag}_jit".lower()
        ctx = dict(module=module, name=name, kind=kind, method=method, dtype=dt, consts=list(spec["consts"]))
        return self._mod(module, ctx, dict(kind=kind)).run(*spec["call"])


def _bind_elementwise(ctx):
    kind, method, consts = ctx["kind"], ctx["method"], ctx["consts"]
    if kind == "map":
        c0 = consts[0] if consts else 0.0
        c1 = consts[1] if len(consts) > 1 else 1.0
        return lambda A: _ffi.map1(method, A, c0, c1).view(A.shape)
    if kind == "map2":
        c1 = consts[0] if consts else 1.0
        return lambda A, B: _ffi.map2(method, A, B, c1).view(A.shape)
    if kind == "map_u8":
        return lambda A, B=None: _ffi.map_u8(method, A, B).view(A.shape)
    if kind == "map_nip":
        return lambda A: _ffi.map_nip(method, A, consts[0]).view(A.shape)
    if kind == "map3":
        return lambda Cnd, A, B: _ffi.where(Cnd, A, B).view(A.shape)
    raise ValueError(f"unknown elementwise kind {kind!r}")


_compile.register_binder(ElementwiseImpl.wrapper_template, _bind_elementwise)

# =============================================================================================
# GEMM family
# =============================================================================================
_SHMEM_BYTES = 101376      # per-block shared memory the reference tiles are sized for
_MAX_THREADS = 1024


def _bt2d_tile(dtype, M, N, K):
    """First SIMT block-tiling plan the reference would pick (kuiops.py:330-362 there), or None.
    Only its existence matters here: it reproduces which shapes the reference accepts."""
    size = dtype.itemsize
    vec = 16 // size
    for bm in (128, 64, 32):
        for bn in (128, 64, 32):
            for bk in (64, 32):
                if M % bm or N % bn or K % bk or bn % vec or bk % vec:
                    continue
                if size * bk * (bm + bn) > _SHMEM_BYTES:
                    continue
                for tm in (16, 8):
                    for tn in (16, 8):
                        if bm % tm or bn % tn:
                            continue
                        threads = (bm // tm) * (bn // tn)
                        if threads > _MAX_THREADS:
                            continue
                        per_pass = vec * threads
                        if (bm * bk) % per_pass == 0 and (bk * bn) % per_pass == 0:
                            return dict(bm=bm, bn=bn, bk=bk, tm=tm, tn=tn)
    return None


def _tc2d_tile(dtype, M, N, K):
    """First wmma tiling plan the reference would pick (kuiops.py:365-394 there), or None."""
    vec = 16 // dtype.itemsize
    frag = 16
    for bm in (128, 64):
        for bn in (128, 64):
            for bk in (64, 32, 16):
                if M % bm or N % bn or K % bk or bn % vec or bk % vec:
                    continue
                if 2 * bk * (bm + bn) > _SHMEM_BYTES:
                    continue
                for wm in (16, 8, 4, 2):
                    for wn in (16, 8, 4, 2):
                        if bm % (frag * wm) or bn % (frag * wn):
                            continue
                        warps = (bm // (wm * frag)) * (bn // (wn * frag))
                        if warps * 32 > _MAX_THREADS:
                            continue
                        per_pass = vec * warps * 32
                        if (bm * bk) % per_pass == 0 and (bk * bn) % per_pass == 0:
                            return dict(bm=bm, bn=bn, bk=bk, tm=frag, tn=frag, tk=frag, wm=wm, wn=wn)
    return None


def _as_gemm_operand(B):
    """(tensor, trans_b): use a `weight.t()` view in place instead of copying it."""
    if B.dim() == 2 and B.stride(0) == 1 and B.stride(1) >= B.shape[0] and B.shape[0] > 1:
        return B.t(), True
    return B, False


class MmImpl(_Family):
    fst_template = "mm/Kuiops.Mm.Inst.fst.j2"
    wrapper_template = "mm/wrapper_mm.cu.j2"
    tune_key = "MM"
    tune_params = {"impl": "tc2d"}
    overloads = (aten.mm.default,)

    def supported(self, func, args, kwargs):
        if len(args) != 2 or kwargs.get("alpha", 1) != 1:
            return None
        A, B = args
        if not (_is_cuda_tensor(A) and _is_cuda_tensor(B) and A.dim() == 2 and B.dim() == 2 and A.dtype == B.dtype):
            return None
        if A.dtype not in _KERNEL_FLOATS:
            return None
        M, K = _ints(A.shape)
        K2, N = _ints(B.shape)
        if K != K2:
            return None
        if C.reference_gates():
            tensor_core = A.dtype in (torch.bfloat16, torch.float16) and self.tune_params.get("impl") == "tc2d"
            tile = _tc2d_tile(A.dtype, M, N, K) if tensor_core else _bt2d_tile(A.dtype, M, N, K)
            if tile is None:
                return None
        elif min(M, N, K) < 1:
            return None
        engine = "tcgen05" if A.dtype != torch.float32 else "simt"
        return (engine, A.dtype, [A, B])

    def tune(self, all_tune_params):
        """Re-time the plans of every GEMM shape recorded so far (``kuipy.tuner``) and hand the table
        back for saving.  Shapes not seen yet are tuned at their first call while ``KUIPY_RE_TUNE``
        is on.  Without a GPU the recorded table is passed through unchanged."""
        from . import tuner
        params = dict(self.tune_params) if isinstance(self.tune_params, dict) else {"impl": "tc2d"}
        plans = dict(params.get("plans", {}))
        if torch.cuda.is_available() and _ffi.is_loadable():
            for key in list(plans):
                try:
                    dt, epi, tb, M, N, K = (int(x) for x in key.split("/"))
                except ValueError:
                    continue
                dtype = {1: torch.bfloat16, 2: torch.float16}.get(dt)
                if dtype is not None:
                    plans[key] = tuner.tune_gemm(dtype, M, N, K, bool(tb), epi)
        params["plans"] = plans
        self.tune_params = params
        all_tune_params[self.tune_key] = params
        return all_tune_params

    def run(self, spec, args, kwargs):
        engine, dt, call = spec
        module = f"Kuiops.Mm.{engine.title()}.{_TAG[dt].title()}"
        ctx = dict(module=module, name="mm_jit", dtype=dt)
        return self._mod(module, ctx, {}).run(*call)


def _bind_mm(ctx):
    def run(A, B):
        Bv, tb = _as_gemm_operand(B)
        if tb:
            return _ffi.gemm(A, Bv, trans_b=True)
        if A.is_contiguous() and B.is_contiguous():
            return _ffi.mm(A, B)                   # reference-order entry point
        return _ffi.gemm(A, B)
    return run


_compile.register_binder(MmImpl.wrapper_template, _bind_mm)


class BmmImpl(_Family):
    fst_template = "bmm/Kuiops.Bmm.Inst.fst.j2"
    wrapper_template = "bmm/wrapper_bmm.cu.j2"
    tune_key = "BMM"
    tune_params = ()
    overloads = (aten.bmm.default,)

    def supported(self, func, args, kwargs):
        if len(args) != 2:
            return None
        A, B = args
        if not (_is_cuda_tensor(A) and _is_cuda_tensor(B) and A.dim() == 3 and B.dim() == 3):
            return None
        if A.dtype != B.dtype or A.dtype not in _KERNEL_FLOATS:
            return None
        Bn, M, K = _ints(A.shape)
        Bn2, K2, N = _ints(B.shape)
        if Bn != Bn2 or K != K2 or min(Bn, M, K, N) < 1:
            return None
        # launch limits of the reference kernel; they also keep every index inside 32 bits
        if M * N > _MAX_NUMEL or max(Bn * M * K, Bn * K * N, Bn * M * N) >= 2 ** 32:
            return None
        return (A.dtype, [A, B])

    def run(self, spec, args, kwargs):
        dt, call = spec
        module = f"Kuiops.Bmm.{_TAG[dt].title()}"
        return self._mod(module, dict(module=module, name="bmm_jit", dtype=dt), {}).run(*call)


_compile.register_binder(BmmImpl.wrapper_template, lambda ctx: (lambda A, B: _ffi.bmm(A, B)))


class AddmmImpl(_Family):
    fst_template = "addmm/Kuiops.Addmm.Inst.fst.j2"
    wrapper_template = "addmm/wrapper_addmm.cu.j2"
    tune_key = "ADDMM"
    tune_params = ()
    overloads = (aten.addmm.default,)

    def supported(self, func, args, kwargs):
        if len(args) != 3:
            return None
        Cin, A, B = args
        if not all(_is_cuda_tensor(t) for t in (Cin, A, B)):
            return None
        if A.dim() != 2 or B.dim() != 2 or not (A.dtype == B.dtype == Cin.dtype) or A.dtype not in _KERNEL_FLOATS:
            return None
        M, K = _ints(A.shape)
        K2, N = _ints(B.shape)
        if K != K2:
            return None
        alpha, beta = _scalar(kwargs.get("alpha", 1)), _scalar(kwargs.get("beta", 1))
        if alpha is None or beta is None:
            return None
        cshape = tuple(_ints(Cin.shape))
        if C.reference_gates():
            # full [M, N] addend only, SIMT tile must exist, M*N within one grid (kuiops.py:526-549 there)
            if Cin.dim() != 2 or cshape != (M, N) or M * N > _MAX_BLOCKS or _bt2d_tile(A.dtype, M, N, K) is None:
                return None
            form = "full"
        else:
            if min(M, N, K) < 1:
                return None
            if cshape == (M, N):
                form = "full"
            elif cshape in ((N,), (1, N)):
                form = "bias"
            else:
                return None
        return (form, A.dtype, M, N, [Cin, A, B], float(alpha), float(beta))

    def run(self, spec, args, kwargs):
        form, dt, M, N, call, alpha, beta = spec
        module = f"Kuiops.Addmm.{form.title()}.{_TAG[dt].title()}"
        ctx = dict(module=module, name="addmm_jit", dtype=dt, form=form)
        return self._mod(module, ctx, {}).run(*call, alpha, beta)


def _bind_addmm(ctx):
    form = ctx["form"]

    def run(Cin, A, B, alpha, beta):
        Bv, tb = _as_gemm_operand(B)
        if form == "bias":
            return _ffi.gemm(A, Bv, trans_b=tb, Cin=Cin.reshape(-1), alpha=alpha, beta=beta)
        if not tb and A.is_contiguous() and B.is_contiguous():
            return _ffi.addmm(Cin, A, B, alpha, beta)      # reference-order entry point, in place on a clone
        return _ffi.gemm(A, Bv, trans_b=tb, Cin=Cin, alpha=alpha, beta=beta)
    return run


_compile.register_binder(AddmmImpl.wrapper_template, _bind_addmm)

# =============================================================================================
# softmax / mean / reduce / topk
# =============================================================================================


class SoftmaxImpl(_Family):
    fst_template = "softmax/Kuiops.Softmax.Inst.fst.j2"
    wrapper_template = "softmax/wrapper_softmax.cu.j2"
    tune_key = "SOFTMAX"
    tune_params = ()
    overloads = (aten._softmax.default,)

    def supported(self, func, args, kwargs):
        if len(args) != 3:
            return None
        X, dim, half_to_float = args
        if not (_is_cuda_tensor(X) and X.dtype in _KERNEL_FLOATS) or half_to_float:
            return None
        rank = X.dim()
        if rank < 1 or _wrap_dim(dim, rank) != rank - 1:
            return None
        n = int(X.shape[-1])
        m = X.numel() // n if n else 0
        if m <= 0 or m > _MAX_BLOCKS or m * n > _MAX_NUMEL:
            return None
        return (X.dtype, m, n, [X])

    def run(self, spec, args, kwargs):
        dt, m, n, call = spec
        module = f"Kuiops.Softmax.{_TAG[dt].title()}"
        X = call[0]
        out = self._mod(module, dict(module=module, name="softmax_jit", dtype=dt), {}).run(X.contiguous().reshape(m, n))
        return out.reshape(X.shape)


# the reference kernel overwrites the caller's clone; here the kernel writes a fresh output
_compile.register_binder(SoftmaxImpl.wrapper_template, lambda ctx: (lambda A2d: _ffi.softmax(A2d)))


class MeanImpl(_Family):
    fst_template = "mean/Kuiops.Mean.Inst.fst.j2"
    wrapper_template = "mean/wrapper_mean.cu.j2"
    tune_key = "MEAN"
    tune_params = ()
    overloads = (aten.mean.dim,)

    def supported(self, func, args, kwargs):
        if len(args) < 2 or kwargs.get("dtype") is not None:
            return None
        X, dim = args[0], args[1]
        keepdim = args[2] if len(args) > 2 else kwargs.get("keepdim", False)
        if not (_is_cuda_tensor(X) and X.dtype in _KERNEL_FLOATS):
            return None
        if not keepdim and C.reference_gates():
            return None
        if isinstance(dim, (list, tuple)):
            if len(dim) != 1:
                return None
            dim = dim[0]
        if dim is None or X.dim() < 1:
            return None
        if _wrap_dim(dim, X.dim()) != X.dim() - 1:
            return None
        n = int(X.shape[-1])
        if n < 1:
            return None
        m = X.numel() // n
        if not (0 < m <= _MAX_BLOCKS) or m * n > _MAX_NUMEL:
            return None
        return (X.dtype, n, bool(keepdim), [X])

    def run(self, spec, args, kwargs):
        dt, n, keepdim, call = spec
        module = f"Kuiops.Mean.{_TAG[dt].title()}.Len{n}"
        out = self._mod(module, dict(module=module, name="mean_jit", dtype=dt, length=n), {}).run(*call)
        return out if keepdim else out.squeeze(-1)


_compile.register_binder(MeanImpl.wrapper_template, lambda ctx: (lambda X: _ffi.mean_lastdim(X)))


class ReduceImpl(_Family):
    """aten.all / aten.any over bool, aten.max over int64 / fp32, to a 0-d tensor.  The reference
    has the kernel (kuiops/reduce/Kuiops.HReducePoly.Exact.fst) but no family; the signatures are
    the ones its checklist records (KERNELS.md:43-45)."""
    fst_template = "reduce/Kuiops.Reduce.Inst.fst.j2"
    wrapper_template = "reduce/wrapper_reduce.cu.j2"
    tune_key = "REDUCE"
    tune_params = ()
    _OPS = {aten.all.default: "all", aten.any.default: "any", aten.max.default: "max"}
    overloads = tuple(_OPS)

    def supported(self, func, args, kwargs):
        if len(args) != 1 or kwargs:
            return None
        X = args[0]
        if not (_is_cuda_tensor(X) and 0 < X.numel() <= _MAX_NUMEL):
            return None
        op = self._OPS.get(func)
        if op in ("all", "any") and X.dtype != torch.bool:
            return None
        if op == "max" and X.dtype not in (torch.int64, torch.float32):
            return None
        return (op, X.dtype, [X])

    def run(self, spec, args, kwargs):
        op, dt, call = spec
        module = f"Kuiops.Reduce.{op.title()}.{_TAG[dt].title()}"
        return self._mod(module, dict(module=module, name="reduce_jit", op=op), {}).run(*call)


_compile.register_binder(ReduceImpl.wrapper_template, lambda ctx: (lambda X, _op=ctx["op"]: _ffi.reduce(_op, X)))


class TopkImpl(_Family):
    """aten.topk(T(2, f32), k) -> (values f32, indices int64) (KERNELS.md:58 of the reference;
    its kuiops/topk/ is empty).  Largest, sorted, last axis; ties by ascending index."""
    fst_template = "topk/Kuiops.Topk.Inst.fst.j2"
    wrapper_template = "topk/wrapper_topk.cu.j2"
    tune_key = "TOPK"
    tune_params = ()
    overloads = (aten.topk.default,)
    MAX_K = 2048

    def supported(self, func, args, kwargs):
        if len(args) < 2:
            return None
        X, k = args[0], args[1]
        dim = args[2] if len(args) > 2 else kwargs.get("dim", -1)
        largest = args[3] if len(args) > 3 else kwargs.get("largest", True)
        if not (_is_cuda_tensor(X) and X.dtype == torch.float32 and X.dim() >= 1 and largest):
            return None
        if _wrap_dim(dim, X.dim()) != X.dim() - 1:
            return None
        n = int(X.shape[-1])
        if not isinstance(k, int) or not (0 < k <= min(n, self.MAX_K)) or X.numel() == 0 or n >= 2 ** 32:
            return None
        return (int(k), [X])

    def run(self, spec, args, kwargs):
        k, call = spec
        module = "Kuiops.Topk.F32"
        return self._mod(module, dict(module=module, name="topk_jit"), {}).run(call[0], k)


_compile.register_binder(TopkImpl.wrapper_template, lambda ctx: (lambda X, k: _ffi.topk(X, k)))

# =============================================================================================
# scaled dot-product attention
# =============================================================================================


class SdpaImpl(_Family):
    """Attention.  "reference" gates: the efficient-attention overload with an explicit additive
    bias, no causal flag, no dropout, equal head counts (kuiops.py:627-660 there, where the family
    is written but not connected).  "wide" gates add the flash-attention and cuDNN-attention
    overloads, causal masking, a missing bias and grouped-query heads."""
    fst_template = "sdpa/Kuiops.Sdpa.Inst.fst.j2"
    wrapper_template = "sdpa/wrapper_sdpa.cu.j2"
    tune_key = "SDPA"
    tune_params = ()
    overloads = (aten._scaled_dot_product_efficient_attention.default,
                 aten._scaled_dot_product_flash_attention.default,
                 aten._scaled_dot_product_cudnn_attention.default)

    def supported(self, func, args, kwargs):
        flash = func is aten._scaled_dot_product_flash_attention.default
        # the cuDNN overload (what ATen picks for bf16 / f16 on this GPU generation) takes the efficient
        # overload's arguments and returns the flash overload's nine values
        cudnn = func is aten._scaled_dot_product_cudnn_attention.default
        if cudnn and C.reference_gates():
            return None
        if flash:
            if C.reference_gates() or len(args) < 3:
                return None
            Q, K, V = args[0], args[1], args[2]
            bias = None
            dropout_p = args[3] if len(args) > 3 else kwargs.get("dropout_p", 0.0)
            is_causal = args[4] if len(args) > 4 else kwargs.get("is_causal", False)
            compute_lse = True
        else:
            if len(args) < 5:
                return None
            Q, K, V, bias, compute_lse = args[0], args[1], args[2], args[3], args[4]
            dropout_p = args[5] if len(args) > 5 else kwargs.get("dropout_p", 0.0)
            is_causal = args[6] if len(args) > 6 else kwargs.get("is_causal", False)
        if dropout_p != 0.0:
            return None
        if C.reference_gates() and (bias is None or is_causal):
            return None
        tensors = (Q, K, V) if bias is None else (Q, K, V, bias)
        if not all(_is_cuda_tensor(t) and t.dim() == 4 for t in tensors):
            return None
        if not all(t.dtype == Q.dtype for t in tensors) or Q.dtype not in _KERNEL_FLOATS:
            return None
        N, H, L, E = _ints(Q.shape)
        N2, Hk, S, E2 = _ints(K.shape)
        N3, Hv, S2, Ev = _ints(V.shape)
        if (N, E) != (N2, E2) or (N, Hk, S) != (N3, Hv, S2) or min(N, H, L, S, E, Ev) < 1:
            return None
        if is_causal and not flash and L != S:
            # the kernels align the causal mask bottom-right (query i sees keys <= i + S - L), which is
            # the flash overload's rule; ATen's efficient overload aligns it top-left, and the two
            # differ whenever the query and key counts do
            return None
        if C.reference_gates():
            if H != Hk or tuple(_ints(bias.shape)) != (N, H, L, S):
                return None
            if L * S > _MAX_NUMEL or L * Ev > _MAX_NUMEL or N * H * L > _MAX_BLOCKS or N * H * L * S > _MAX_NUMEL:
                return None
            if max(N * H * L * E, N * H * S * E, N * H * S * Ev, N * H * L * Ev, N * H * L * S) >= 2 ** 32:
                return None
        else:
            if Hk < 1 or H % Hk or Ev > 256 or E > 1024:
                return None
            if bias is not None:
                try:
                    if tuple(torch.broadcast_shapes(tuple(bias.shape), (N, H, L, S))) != (N, H, L, S):
                        return None
                except RuntimeError:
                    return None
        scale = kwargs.get("scale")
        if scale is None:
            scale = 1.0 / math.sqrt(E)
        return (Q.dtype, float(scale), bool(is_causal), "flash" if flash else ("cudnn" if cudnn else "efficient"),
                bool(compute_lse), [Q, K, V, bias])

    def run(self, spec, args, kwargs):
        dt, scale, causal, overload, compute_lse, call = spec
        module = f"Kuiops.Sdpa.{_TAG[dt].title()}"
        Q, K, V, bias = call
        out, lse = self._mod(module, dict(module=module, name="sdpa_jit", dtype=dt), {}).run(Q, K, V, bias, scale, causal)
        zero = torch.empty([], dtype=torch.int64)
        if overload == "efficient":
            # aten returns (output, log_sumexp f32, philox_seed, philox_offset)
            return (out, lse, zero, zero)
        L, S = int(Q.shape[2]), int(K.shape[2])
        # (output, logsumexp, cum_seq_q, cum_seq_k, max_q, max_k, philox_seed, philox_offset, debug_attn_mask)
        if overload == "cudnn":
            return (out, lse.unsqueeze(-1), None, None, L, S, zero, zero, None)     # its log-sum-exp is (N, H, L, 1)
        empty = torch.empty(0, dtype=dt, device=Q.device)
        return (out, lse, None, None, L, S, zero, zero, empty)


def _bind_sdpa(ctx):
    def run(Q, K, V, bias, scale, causal=False):
        return _ffi.sdpa(Q, K, V, bias=bias, scale=scale, is_causal=causal, need_lse=True)
    return run


_compile.register_binder(SdpaImpl.wrapper_template, _bind_sdpa)

# =============================================================================================
# indexed data movement
# =============================================================================================
_PAYLOAD_SIZES = (1, 2, 4, 8)


class GatherImpl(_Family):
    fst_template = "gather/Kuiops.Gather.Inst.fst.j2"
    wrapper_template = "gather/wrapper_gather.cu.j2"
    tune_key = "GATHER"
    tune_params = ()
    overloads = (aten.gather.default,)

    def supported(self, func, args, kwargs):
        if len(args) < 3 or kwargs.get("sparse_grad", False):
            return None
        Inp, dim, Idx = args[0], args[1], args[2]
        if not (_is_cuda_tensor(Inp) and _is_cuda_tensor(Idx)) or Idx.dtype != torch.int64:
            return None
        rank = Inp.dim()
        if rank < 1 or rank > 8 or Idx.dim() != rank or Inp.element_size() not in _PAYLOAD_SIZES:
            return None
        dim = _wrap_dim(dim, rank)
        if not 0 <= dim < rank:
            return None
        ishape, xshape = _ints(Inp.shape), _ints(Idx.shape)
        if C.reference_gates():
            if not _pointwise_le(xshape, ishape):         # `shape_le idx inp` on every axis
                return None
        elif any(xshape[d] > ishape[d] for d in range(rank) if d != dim):
            return None
        if not 0 < _prod(xshape) <= _MAX_NUMEL:
            return None
        return (Inp.dtype, dim, ishape, xshape, [Inp, Idx])

    def run(self, spec, args, kwargs):
        dt, dim, ishape, xshape, call = spec
        module = f"Kuiops.Gather.{_TAG.get(dt, 'b' + str(dt.itemsize)).title()}.R{len(ishape)}.Dim{dim}"
        return self._mod(module, dict(module=module, name="gather_jit", dim=dim, r=len(ishape)), {}).run(*call)


_compile.register_binder(GatherImpl.wrapper_template,
                         lambda ctx: (lambda Inp, Idx, _d=ctx["dim"]: _ffi.gather(Inp, _d, Idx)))


class ScatterImpl(_Family):
    fst_template = "scatter/Kuiops.Scatter.Inst.fst.j2"
    wrapper_template = "scatter/wrapper_scatter.cu.j2"
    tune_key = "SCATTER"
    tune_params = ()
    overloads = (aten.scatter.src,)

    def supported(self, func, args, kwargs):
        if len(args) < 4:
            return None
        Self, dim, Idx, Src = args[0], args[1], args[2], args[3]
        if not all(_is_cuda_tensor(t) for t in (Self, Idx, Src)):
            return None
        if Src.dtype != Self.dtype or Idx.dtype != torch.int64 or Self.element_size() not in _PAYLOAD_SIZES:
            return None
        rank = Self.dim()
        if rank < 1 or rank > 8 or Idx.dim() != rank or Src.dim() != rank:
            return None
        dim = _wrap_dim(dim, rank)
        if not 0 <= dim < rank:
            return None
        self_shape, idx_shape, src_shape = _ints(Self.shape), _ints(Idx.shape), _ints(Src.shape)
        # the kernel walks one shape for src and index, pointwise inside self's
        if src_shape != idx_shape or not _pointwise_le(src_shape, self_shape):
            return None
        if not 0 < _prod(src_shape) <= _MAX_NUMEL:
            return None
        return (Self.dtype, dim, src_shape, self_shape, [Self, Idx, Src])

    def run(self, spec, args, kwargs):
        dt, dim, src_shape, self_shape, call = spec
        module = f"Kuiops.Scatter.{_TAG.get(dt, 'b' + str(dt.itemsize)).title()}.R{len(self_shape)}.Dim{dim}"
        return self._mod(module, dict(module=module, name="scatter_jit", dim=dim, r=len(self_shape)), {}).run(*call)


_compile.register_binder(ScatterImpl.wrapper_template,
                         lambda ctx: (lambda Self, Idx, Src, _d=ctx["dim"]: _ffi.scatter(Self, _d, Idx, Src)))


class CatImpl(_Family):
    fst_template = "cat/Kuiops.Cat.Inst.fst.j2"
    wrapper_template = "cat/wrapper_cat.cu.j2"
    tune_key = "CAT"
    tune_params = ()
    overloads = (aten.cat.default,)

    def supported(self, func, args, kwargs):
        if len(args) < 1:
            return None
        tensors = args[0]
        dim = args[1] if len(args) > 1 else kwargs.get("dim", 0)
        if not isinstance(tensors, (list, tuple)) or len(tensors) < 2:
            return None
        if C.reference_gates() and len(tensors) != 2:      # the reference kernel is binary
            return None
        if not all(_is_cuda_tensor(t) for t in tensors):
            return None
        first = tensors[0]
        rank = first.dim()
        if rank < 1 or rank > 8 or first.element_size() not in _PAYLOAD_SIZES:
            return None
        if any(t.dtype != first.dtype or t.dim() != rank for t in tensors):
            return None
        dim = _wrap_dim(dim, rank)
        if not 0 <= dim < rank:
            return None
        base = _ints(first.shape)
        for t in tensors[1:]:
            if any(int(t.shape[d]) != base[d] for d in range(rank) if d != dim):
                return None
        out_shape = list(base)
        out_shape[dim] = sum(int(t.shape[dim]) for t in tensors)
        if not 0 < _prod(out_shape) <= _MAX_NUMEL:
            return None
        return (first.dtype, dim, out_shape, list(tensors))

    def run(self, spec, args, kwargs):
        dt, dim, out_shape, call = spec
        arity = "Binary" if len(call) == 2 else "Nary"
        module = f"Kuiops.Cat.{arity}.{_TAG.get(dt, 'b' + str(dt.itemsize)).title()}.R{len(out_shape)}.Dim{dim}"
        return self._mod(module, dict(module=module, name="cat_jit", dim=dim, r=len(out_shape)), {}).run(*call)


def _bind_cat(ctx):
    dim = ctx["dim"]

    def run(*tensors):
        if len(tensors) == 2:
            return _ffi.cat2(tensors[0], tensors[1], dim)     # reference-order entry point
        return _ffi.cat(tensors, dim)
    return run


_compile.register_binder(CatImpl.wrapper_template, _bind_cat)


class IndexImpl(_Family):
    """aten.index.Tensor with int64 index tensors on adjacent dims (None before and after), e.g.
    ``mask[i, j]`` with broadcast 4-d indices (KERNELS.md:67 of the reference) or ``ids[:, pos]``."""
    fst_template = "index/Kuiops.Index.Inst.fst.j2"
    wrapper_template = "index/wrapper_index.cu.j2"
    tune_key = "INDEX"
    tune_params = ()
    overloads = (aten.index.Tensor,)

    def supported(self, func, args, kwargs):
        if len(args) != 2:
            return None
        Self, indices = args
        if not _is_cuda_tensor(Self) or not isinstance(indices, (list, tuple)) or not indices:
            return None
        if Self.element_size() not in _PAYLOAD_SIZES or not 1 <= Self.dim() <= 8 or len(indices) > Self.dim():
            return None
        used = [i for i, t in enumerate(indices) if t is not None]
        if not used or used != list(range(used[0], used[-1] + 1)) or len(used) > 4:
            return None
        idx = [indices[i] for i in used]
        if not all(_is_cuda_tensor(t) and t.dtype == torch.int64 for t in idx):
            return None
        try:
            bshape = torch.broadcast_shapes(*[tuple(t.shape) for t in idx])
        except RuntimeError:
            return None
        if len(bshape) > 8 or Self.numel() == 0 or _prod(bshape) == 0:
            return None
        return (Self.dtype, used[0], idx, [Self])

    def run(self, spec, args, kwargs):
        dt, first, idx, call = spec
        module = f"Kuiops.Index.{_TAG.get(dt, 'b' + str(dt.itemsize)).title()}.R{call[0].dim()}.At{first}.N{len(idx)}"
        return self._mod(module, dict(module=module, name="index_jit", first=first), {}).run(call[0], idx)


_compile.register_binder(IndexImpl.wrapper_template,
                         lambda ctx: (lambda Self, idx, _f=ctx["first"]: _ffi.index(Self, _f, idx)))


class IsinImpl(_Family):
    """aten.isin(int64 elements, int64 test set or 0-d) -> bool (KERNELS.md:56-57 of the reference)."""
    fst_template = "isin/Kuiops.Isin.Inst.fst.j2"
    wrapper_template = "isin/wrapper_isin.cu.j2"
    tune_key = "ISIN"
    tune_params = ()
    overloads = (aten.isin.Tensor_Tensor,)

    def supported(self, func, args, kwargs):
        if len(args) < 2:
            return None
        E, T = args[0], args[1]
        invert = kwargs.get("invert", args[3] if len(args) > 3 else False)
        if not (_is_cuda_tensor(E) and _is_cuda_tensor(T)):
            return None
        if E.dtype != torch.int64 or T.dtype != torch.int64 or E.numel() == 0:
            return None
        return (bool(invert), [E, T])

    def run(self, spec, args, kwargs):
        invert, call = spec
        module = "Kuiops.Isin.I64"
        return self._mod(module, dict(module=module, name="isin_jit"), {}).run(*call, invert)


_compile.register_binder(IsinImpl.wrapper_template, lambda ctx: (lambda E, T, inv=False: _ffi.isin(E, T, inv)))


class DataMoveImpl(_Family):
    """The data-movement ops a decoder issues next to its compute on every token: dtype casts
    (aten._to_copy between float types), aten.clone, aten.masked_fill.Scalar, aten.argmax,
    aten.cumsum and aten.sort over the last axis, aten.multinomial (one draw per row, or several with
    replacement, from a documented Philox stream) and aten.embedding.  The reference lists them as backlog without kernels
    (KERNELS.md:46-48,68-90); dense, contiguous operands only, everything else falls through."""
    fst_template = "datamove/Kuiops.DataMove.Inst.fst.j2"
    wrapper_template = "datamove/wrapper_datamove.cu.j2"
    tune_key = "DATAMOVE"
    tune_params = ()
    _FLOATS = (torch.float32, torch.bfloat16, torch.float16)
    overloads = (aten._to_copy.default, aten.clone.default, aten.masked_fill.Scalar, aten.argmax.default,
                 aten.cumsum.default, aten.sort.default, aten.sort.stable, aten.embedding.default, aten.multinomial.default)

    @staticmethod
    def _dense(X):
        return _is_cuda_tensor(X) and X.is_contiguous() and 0 < X.numel() <= _MAX_NUMEL

    def supported(self, func, args, kwargs):
        if not args:
            return None
        X = args[0]
        if func is aten._to_copy.default:
            dt = kwargs.get("dtype") or X.dtype
            dev = kwargs.get("device")
            same_gpu = dev is None or (torch.device(dev).type == "cuda" and torch.device(dev) == X.device)
            plain = (same_gpu and kwargs.get("layout") in (None, torch.strided)
                     and not kwargs.get("pin_memory") and kwargs.get("memory_format") in (None, torch.preserve_format, torch.contiguous_format))
            if len(args) == 1 and self._dense(X) and plain and X.dtype in self._FLOATS and dt in self._FLOATS:
                return ("cast", dt, [X])
            return None
        if func is aten.clone.default:
            fmt = kwargs.get("memory_format", args[1] if len(args) > 1 else None)
            if self._dense(X) and X.dtype in self._FLOATS and fmt in (None, torch.preserve_format, torch.contiguous_format):
                return ("cast", X.dtype, [X])
            return None
        if func is aten.masked_fill.Scalar:
            if len(args) != 3 or kwargs:
                return None
            M, v = args[1], args[2]
            if (self._dense(X) and X.dtype in self._FLOATS and self._dense(M) and M.dtype == torch.bool
                    and tuple(M.shape) == tuple(X.shape) and isinstance(v, (int, float)) and not isinstance(v, bool)):
                return ("masked_fill", float(v), [X, M])
            return None
        if func is aten.argmax.default:
            dim = kwargs.get("dim", args[1] if len(args) > 1 else None)
            keep = kwargs.get("keepdim", args[2] if len(args) > 2 else False)
            if (self._dense(X) and X.dtype in self._FLOATS and X.dim() >= 1 and dim is not None and not keep
                    and _wrap_dim(dim, X.dim()) == X.dim() - 1):
                return ("argmax", None, [X])
            return None
        if func is aten.cumsum.default:
            dim = kwargs.get("dim", args[1] if len(args) > 1 else None)
            dt = kwargs.get("dtype", args[2] if len(args) > 2 else None)
            if (self._dense(X) and X.dtype in (torch.float32, torch.int64) and X.dim() >= 1 and isinstance(dim, int)
                    and _wrap_dim(dim, X.dim()) == X.dim() - 1 and dt in (None, X.dtype)):
                return ("cumsum", None, [X])
            return None
        if func is aten.sort.default or func is aten.sort.stable:
            # sort.default(self, dim=-1, descending=False); sort.stable(self, *, stable, dim=-1, descending=False).
            # The kernel is stable, which also satisfies a call that does not ask for it.
            if func is aten.sort.default:
                dim = kwargs.get("dim", args[1] if len(args) > 1 else -1)
                desc = kwargs.get("descending", args[2] if len(args) > 2 else False)
                extra = len(args) > 3
            else:
                dim, desc, extra = kwargs.get("dim", -1), kwargs.get("descending", False), len(args) > 1
            if (not extra and self._dense(X) and X.dtype == torch.float32 and X.dim() >= 1 and isinstance(dim, int)
                    and isinstance(desc, bool) and _wrap_dim(dim, X.dim()) == X.dim() - 1):
                return ("sort", desc, [X])
            return None
        if func is aten.multinomial.default:
            # multinomial(self, num_samples, replacement=False, *, generator=None): one draw per row, or several
            # independent ones; draws without replacement depend on each other and stay with PyTorch
            k = args[1] if len(args) > 1 else kwargs.get("num_samples")
            repl = kwargs.get("replacement", args[2] if len(args) > 2 else False)
            gen = kwargs.get("generator")
            if (self._dense(X) and X.dtype == torch.float32 and X.dim() in (1, 2) and isinstance(k, int) and not isinstance(k, bool)
                    and 1 <= k <= 4096 and (k == 1 or repl) and (gen is None or gen.device.type == "cuda")):
                return ("multinomial", (k, gen), [X])
            return None
        if func is aten.embedding.default:
            if len(args) < 2:
                return None
            ids = args[1]
            extra = list(args[2:]) + list(kwargs.values())
            if any(bool(e) and e != -1 for e in extra[1:]):          # scale_grad_by_freq / sparse
                return None
            if (self._dense(X) and X.dim() == 2 and X.dtype in self._FLOATS and _is_cuda_tensor(ids) and ids.dtype == torch.int64
                    and ids.numel() > 0):
                return ("embedding", None, [X, ids])
            return None
        return None

    def run(self, spec, args, kwargs):
        op, extra, call = spec
        module = f"Kuiops.DataMove.{op.title().replace('_', '')}"
        return self._mod(module, dict(module=module, name="datamove_jit", op=op), {}).run(*call, extra)


def _datamove_binder(ctx):
    op = ctx["op"]
    if op == "cast":
        return lambda X, dt: _ffi.cast(X, dt)
    if op == "masked_fill":
        return lambda X, M, v: _ffi.masked_fill(X, M, v)
    if op == "argmax":
        return lambda X, _=None: _ffi.argmax_lastdim(X)
    if op == "cumsum":
        return lambda X, _=None: _ffi.cumsum_lastdim(X)
    if op == "sort":
        return lambda X, desc: _ffi.sort_lastdim(X, desc)
    if op == "multinomial":
        def draw(X, extra):
            # the stream position comes from (and is advanced in) the CUDA generator the call names, or the
            # device's default one: seed = its seed, offset = its Philox offset, moved on by 4 per call
            k, gen = extra
            if gen is None:
                gen = torch.cuda.default_generators[X.device.index if X.device.index is not None else torch.cuda.current_device()]
            off = gen.get_offset()
            gen.set_offset(off + 4)
            return _ffi.multinomial(X, k, gen.initial_seed(), off)
        return draw
    return lambda W, ids, _=None: _ffi.embedding(W, ids)


_compile.register_binder(DataMoveImpl.wrapper_template, _datamove_binder)

