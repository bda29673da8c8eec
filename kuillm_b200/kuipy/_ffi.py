"""ctypes binding of ``libkuiops.so`` (the C ABI declared in ``include/kuiops.h``).

This is the only place that touches the shared library.  It plays the part of the reference's
generated pybind wrappers (kuiops/<op>/wrapper_<op>.cu.j2): make inputs contiguous, allocate the
output with the kernel's output dtype, pass raw pointers, sizes and the current CUDA stream.
Unlike those wrappers it never synchronises the stream (include/kuiops.h:11-18 of the reference
does before every launch), and there is no CPU path: if the library cannot be loaded, every call
raises.
"""
import ctypes
import os
from pathlib import Path

import torch

from . import config as _C

_PKG = Path(__file__).resolve().parent.parent
LIB_PATH = Path(os.environ.get("KUIOPS_LIB", _PKG / "lib" / "libkuiops.so"))

OK, EINVAL, EUNSUPPORTED, EWORKSPACE, ELAUNCH, EDRIVER, ELIMIT = 0, -1, -2, -3, -4, -5, -6
F32, BF16, F16 = 0, 1, 2
GEMM_COUNTER_BYTES = 16384
SDPA_NOALLOC_SCRATCH_BYTES = 8 << 20
REDUCE_WORKSPACE_BYTES = 16384
REDUCE_ALL, REDUCE_ANY, REDUCE_MAX = 0, 1, 2
MAP = dict(silu=0, neg=1, rsqrt=2, cos=3, sin=4, pow=5, square=6, add=7, mul=8, sub=9, div=10,
           bnot=11, band=12, bor=13, eq=14, le=15, lt=16, gelu=17)

_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}


class KuiopsError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        super().__init__(f"{what}: {strerror(code)} (code {code})")


_lib = None
_load_error = None

c_void_p, c_int, c_u32, c_u64, c_i64, c_float, c_double, c_size_t = (
    ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int64,
    ctypes.c_float, ctypes.c_double, ctypes.c_size_t)
_P64 = ctypes.POINTER(ctypes.c_uint64)
_PI64 = ctypes.POINTER(ctypes.c_int64)
_PP = ctypes.POINTER(ctypes.c_void_p)

# name -> (restype, argtypes); mirrors include/kuiops.h declaration by declaration
SIGNATURES = {
    "kuiops_abi_version": (c_int, []),
    "kuiops_strerror": (ctypes.c_char_p, [c_int]),
    "kuiops_debug_tc_error": (c_int, [ctypes.POINTER(ctypes.c_uint), c_int]),
    "kuiops_debug_set_peer_wait_ns": (c_u64, [c_u64]),
    "kuiops_debug_gemm_trace": (c_int, [c_void_p]),
    "kuiops_launch_count": (c_u64, []),
    "kuiops_set_pdl": (c_int, [c_int]),
    "kuiops_gemm_workspace_bytes": (c_size_t, [c_int, c_u32, c_u32, c_u32, c_u32]),
    "kuiops_gemm_tune_set": (c_int, [c_int, c_int, c_int, c_u32, c_u32, c_u32, c_int, c_int]),
    "kuiops_gemm_tune_clear": (c_int, []),
    "kuiops_gemm_set_sm_reserve": (c_int, [c_int]),
    "kuiops_gemm_tune_query": (c_int, [c_int, c_int, c_int, c_u32, c_u32, c_u32, ctypes.POINTER(c_int), ctypes.POINTER(c_int),
                                       ctypes.POINTER(c_int)]),
    "kuiops_gemm": (c_int, [c_int, c_int, c_u32, c_u32, c_u32, c_u32,
                            c_void_p, c_i64, c_i64, c_void_p, c_i64, c_i64, c_int,
                            c_void_p, c_i64, c_i64, c_float, c_float,
                            c_void_p, c_i64, c_i64, c_void_p, c_size_t, c_void_p]),
    "kuiops_gemm_swiglu": (c_int, [c_int, c_u32, c_u32, c_u32, c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_i64,
                                   c_void_p, c_size_t, c_void_p]),
    "kuiops_gemm_rope_qkv": (c_int, [c_int, c_u32, c_u32, c_u32, c_u32, c_u32, c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_i64,
                                     c_void_p, c_float, c_void_p, c_void_p, c_u64, c_u32, c_void_p]),
    "kuiops_gemm_residual_ssq": (c_int, [c_int, c_u32, c_u32, c_u32, c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_void_p]),
    "kuiops_gemm_swiglu_rms": (c_int, [c_int, c_u32, c_u32, c_u32, c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_i64,
                                       c_void_p, c_u32, c_float, c_void_p]),
    "kuiops_gemm_rope_qkv_rms": (c_int, [c_int, c_u32, c_u32, c_u32, c_u32, c_u32, c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_i64,
                                         c_void_p, c_float, c_void_p, c_void_p, c_u64, c_u32, c_void_p, c_u32, c_float, c_void_p]),
    "kuiops_gemm_push": (c_int, [c_int, c_u32, c_u32, c_u32, c_void_p, c_i64, c_void_p, c_i64, c_int, c_u32, c_u32, _P64,
                                 c_u64, c_void_p, c_void_p]),
    "kuiops_rmsnorm_gather": (c_int, [c_int, c_u64, c_u32, c_u32, c_void_p, c_u64, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_float, c_void_p, c_void_p, c_void_p]),
    "kuiops_debug_sdpa_splits": (c_int, [c_int]),
    "kuiops_sdpa_workspace_bytes": (c_size_t, [c_int] + [c_u32] * 7),
    "kuiops_sdpa": (c_int, [c_int] + [c_u32] * 7 +
                    [c_void_p, c_i64, c_i64, c_i64] * 3 +
                    [c_void_p, c_float, c_int, c_void_p, c_i64, c_i64, c_i64, c_void_p,
                     c_void_p, c_size_t, c_void_p]),
    "kuiops_sdpa_varlen": (c_int, [c_int] + [c_u32] * 7 +
                           [c_void_p, c_i64, c_i64, c_i64] * 3 +
                           [c_void_p, c_float, c_int, c_void_p, c_i64, c_i64, c_i64, c_void_p, c_void_p,
                            c_void_p, c_size_t, c_void_p]),
    "kuiops_sdpa_noalloc": (c_int, [c_int] + [c_u32] * 7 +
                            [c_void_p, c_i64, c_i64, c_i64] * 3 +
                            [c_void_p, c_float, c_int, c_void_p, c_i64, c_i64, c_i64, c_void_p, c_void_p, c_void_p]),
    "kuiops_add_i64": (c_int, [c_u64, c_void_p, c_i64, c_void_p]),
    "kuiops_topk_f32": (c_int, [c_u32, c_u32, c_u32, c_void_p, c_void_p, c_void_p, c_void_p]),
    "kuiops_gather": (c_int, [c_u32, c_u32, c_u32, _P64, _P64, c_void_p, c_void_p, c_void_p, c_u64,
                              c_void_p, c_void_p]),
    "kuiops_scatter": (c_int, [c_u32, c_u32, c_u32, _P64, _P64, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_u64, c_void_p, c_void_p]),
    "kuiops_cat": (c_int, [c_u32, c_u32, c_u32, _P64, c_u64, c_void_p, c_void_p, c_void_p, c_u64, c_void_p]),
    "kuiops_cat_n": (c_int, [c_u32, c_u32, c_u32, c_u32, _P64, _P64, _PP, c_void_p, c_void_p]),
    "kuiops_index": (c_int, [c_u32, c_u32, _P64, c_u32, c_u32, _PP, c_u32, _P64, _PI64,
                             c_void_p, c_void_p, c_void_p, c_void_p]),
    "kuiops_isin_i64": (c_int, [c_u64, c_void_p, c_u64, c_void_p, c_int, c_void_p, c_void_p]),
    "kuiops_map": (c_int, [c_int, c_int, c_u64, c_void_p, c_void_p, c_double, c_double, c_void_p]),
    "kuiops_map2": (c_int, [c_int, c_int, c_u64, c_void_p, c_void_p, c_void_p, c_double, c_void_p]),
    "kuiops_map_u8": (c_int, [c_int, c_u64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "kuiops_map_nip": (c_int, [c_int, c_int, c_u64, c_void_p, c_void_p, c_double, c_void_p]),
    "kuiops_map3": (c_int, [c_u32, c_u64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "kuiops_rmsnorm": (c_int, [c_int, c_u64, c_u32, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
                               c_void_p, c_void_p]),
    "kuiops_swiglu": (c_int, [c_int, c_u64, c_u32, c_void_p, c_void_p, c_void_p]),
    "kuiops_rope_qkv": (c_int, [c_int, c_u64, c_u32, c_u32, c_u32, c_void_p, c_i64, c_void_p, c_float,
                                c_void_p, c_void_p, c_u64, c_u32, c_void_p]),
    "kuiops_cast": (c_int, [c_int, c_int, c_u64, c_void_p, c_void_p, c_void_p]),
    "kuiops_masked_fill": (c_int, [c_int, c_u64, c_void_p, c_void_p, c_double, c_void_p, c_void_p]),
    "kuiops_embedding": (c_int, [c_u32, c_u64, c_u64, c_u64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "kuiops_cumsum_f32": (c_int, [c_u32, c_u32, c_void_p, c_void_p, c_void_p]),
    "kuiops_cumsum_i64": (c_int, [c_u32, c_u32, c_void_p, c_void_p, c_void_p]),
    "kuiops_sort_workspace_bytes": (c_size_t, [c_u32, c_u32]),
    "kuiops_sort_f32": (c_int, [c_u32, c_u32, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "kuiops_multinomial_f32": (c_int, [c_u32, c_u32, c_u32, c_void_p, c_void_p, c_u64, c_u64, c_void_p, c_void_p]),
    "kuiops_argmax": (c_int, [c_int, c_u64, c_u64, c_void_p, c_void_p, c_void_p]),
    "kuiops_sample_workspace_bytes": (c_size_t, [c_u32, c_u32]),
    "kuiops_sample_topk_topp_f32": (c_int, [c_u32, c_u32, c_void_p, c_float, c_u32, c_float, c_u64, c_u64, c_void_p, c_void_p,
                                            c_void_p, c_size_t, c_void_p]),
}
for _sfx in ("f32", "bf16", "f16"):
    SIGNATURES[f"kuiops_mm_{_sfx}"] = (c_int, [c_u32, c_u32, c_u32, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_size_t, c_void_p])
    SIGNATURES[f"kuiops_addmm_{_sfx}"] = (c_int, [c_u32, c_u32, c_u32, c_float, c_float, c_void_p, c_void_p,
                                                  c_void_p, c_void_p, c_size_t, c_void_p])
    SIGNATURES[f"kuiops_bmm_{_sfx}"] = (c_int, [c_u32, c_u32, c_u32, c_u32, c_void_p, c_void_p, c_void_p,
                                                c_void_p, c_size_t, c_void_p])
    SIGNATURES[f"kuiops_softmax_{_sfx}"] = (c_int, [c_u32, c_u32, c_void_p, c_void_p, c_void_p])
    SIGNATURES[f"kuiops_mean_{_sfx}"] = (c_int, [c_u64, c_u64, c_void_p, c_void_p, c_void_p])
for _sfx in ("u8", "i64", "f32"):
    SIGNATURES[f"kuiops_reduce_{_sfx}"] = (c_int, [c_int, c_u64, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p])


def lib():
    """The loaded library.  Raises if it is missing: there is no fallback path."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    if _load_error is not None:
        raise _load_error
    try:
        if not LIB_PATH.exists():
            raise OSError(f"{LIB_PATH} not found; build it with `python {_PKG / 'csrc' / 'build.py'}`")
        L = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
        try:
            # tuned GEMM plans: the table shipped with the package, then the user's own (KUIPY_CACHE)
            from . import tuner
            tuner.apply(tuner.load_tables(), L)
        except Exception as e:      # noqa: BLE001 - a damaged table must not make the kernels unavailable
            _C.log(f"tuned plans not applied: {e}")
        return L
    except (OSError, AttributeError) as e:
        _load_error = RuntimeError(f"kuiops: cannot load the CUDA library: {e}")
        raise _load_error


def is_loadable() -> bool:
    try:
        lib()
        return True
    except RuntimeError:
        return False


def strerror(code: int) -> str:
    try:
        return lib().kuiops_strerror(code).decode()
    except RuntimeError:
        return f"kuiops error {code}"


def gemm_plan(dtype, M, N, K, trans_b=True, epilogue=0):
    """(splits, column tile, swapped placement) the tcgen05 GEMM would run this shape with."""
    s, b, w = c_int(0), c_int(0), c_int(0)
    _check(lib().kuiops_gemm_tune_query(dtype_code(dtype), epilogue, 1 if trans_b else 0, M, N, K, ctypes.byref(s), ctypes.byref(b),
                                        ctypes.byref(w)), "gemm_tune_query")
    return s.value, b.value, bool(w.value)


def gemm_set_sm_reserve(sms: int) -> int:
    """SMs the persistent GEMM leaves free for kernels of other streams (0 = none); returns the old setting."""
    return int(lib().kuiops_gemm_set_sm_reserve(int(sms)))


def set_pdl(enabled: bool) -> bool:
    """Turn programmatic dependent launch of the decode-path kernels on or off; returns the old setting."""
    return bool(lib().kuiops_set_pdl(1 if enabled else 0))


def set_peer_wait_ns(ns: int) -> int:
    """Limit of the cross-GPU flag wait of rmsnorm_gather (0 = the default two seconds); returns the old limit."""
    return int(lib().kuiops_debug_set_peer_wait_ns(int(ns)))


def launch_count() -> int:
    return int(lib().kuiops_launch_count())


def tc_error(reset=True) -> int:
    v = ctypes.c_uint(0)
    _check(lib().kuiops_debug_tc_error(ctypes.byref(v), 1 if reset else 0), "debug_tc_error")
    if v.value:
        drop_workspaces()      # a kernel gave up mid-way: its ticket words may be non-zero
    return int(v.value)


def _check(rc, what):
    if rc != OK:
        if rc in (ELAUNCH, EDRIVER):
            drop_workspaces()
        raise KuiopsError(rc, what)


def _ptr(t):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_cur_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """Handle of the current device's current stream (the raw getters cost a tenth of the Stream object)."""
    if _raw_stream is not None and _cur_device is not None:
        return _raw_stream(_cur_device())
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dt):
    try:
        return _DT[dt]
    except KeyError:
        raise KuiopsError(EINVAL, f"dtype {dt}")


def _sfx(dt):
    return {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}[dt]


def _u64arr(vals):
    return (ctypes.c_uint64 * len(vals))(*[int(v) for v in vals])


# --------------------------------------------------------------------------------------------
# caller-owned scratch: one zero-initialised buffer per (purpose, device, stream); the kernels
# keep the leading counter words zero between calls
# --------------------------------------------------------------------------------------------
_scratch = {}


def drop_workspaces():
    """Forget every cached scratch buffer.  The kernels only restore "ticket words are zero" when
    they run to completion; after a timed-out wait or a failed launch the next call gets a fresh,
    zero-initialised buffer instead of one whose counters may be half-way."""
    _scratch.clear()


def workspace(kind, device, nbytes):
    key = (kind, device.index if device.index is not None else torch.cuda.current_device(), _stream())
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        cap = max(int(nbytes), 1 << 20)
        buf = torch.zeros(cap, dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


# --------------------------------------------------------------------------------------------
# GEMM family
# --------------------------------------------------------------------------------------------
def gemm(A, B, *, trans_b=False, Cin=None, alpha=1.0, beta=1.0, out=None, out_dtype=None):
    """C = alpha * A @ (B.T if trans_b else B) + beta * Cin.  A: [M,K] or [b,M,K].
    B: [K,N] ([N,K] if trans_b), optionally batched.  Cin: [M,N], [b,M,N] or a length-N bias."""
    batched = A.dim() == 3
    if batched:
        bsz, M, K = A.shape
    else:
        bsz, (M, K) = 1, A.shape
    N = B.shape[-2] if trans_b else B.shape[-1]
    dt = A.dtype
    odt = out_dtype or dt
    if A.stride(-1) != 1 or (batched and A.stride(0) < M * A.stride(1) and bsz > 1):
        A = A.contiguous()
    if B.stride(-1) != 1:
        B = B.contiguous()
    lda, ldb = A.stride(-2), B.stride(-2)
    if M == 1:
        lda = max(lda, K)
    if (K if not trans_b else N) == 1:
        ldb = max(ldb, K if trans_b else N)
    sa = A.stride(0) if batched else 0
    sb = B.stride(0) if B.dim() == 3 else 0
    if out is None:
        out = torch.empty((bsz, M, N) if batched else (M, N), dtype=odt, device=A.device)
    ldc, sc = out.stride(-2), (out.stride(0) if batched else 0)
    if M == 1:
        ldc = max(ldc, N)
    cin_p, ldcin, scin = None, 0, 0
    if Cin is not None:
        if Cin.dim() == 1:
            Cin = Cin.contiguous()
            cin_p, ldcin, scin = Cin.data_ptr(), 0, 0
        else:
            if Cin.stride(-1) != 1:
                Cin = Cin.contiguous()
            cin_p, ldcin = Cin.data_ptr(), max(Cin.stride(-2), N)
            scin = Cin.stride(0) if Cin.dim() == 3 else 0
    L = lib()
    code = dtype_code(dt)
    if _C.RE_TUNE and not batched:
        from . import tuner
        tuner.maybe_tune(dt, M, N, K, trans_b, 0)
    wsb = L.kuiops_gemm_workspace_bytes(code, bsz, M, N, K)
    ws = workspace("gemm", A.device, wsb)
    _check(L.kuiops_gemm(code, dtype_code(odt), bsz, M, N, K,
                         A.data_ptr(), lda, sa, B.data_ptr(), ldb, sb, 1 if trans_b else 0,
                         cin_p, ldcin, scin, float(alpha), float(beta),
                         out.data_ptr(), ldc, sc, ws.data_ptr(), ws.numel(), _stream()), "gemm")
    return out


def gemm_rope_qkv(A, W, hq, hk, d, positions, theta, k_cache=None, v_cache=None, rows_per_seq=1, out=None):
    """Packed QKV projection with the rotary embedding and the KV-cache append in the GEMM's epilogue;
    None when the shape does not suit the fused kernel (the caller then runs gemm + rope_qkv)."""
    M, K = A.shape
    N = (hq + 2 * hk) * d
    if A.dtype not in (torch.bfloat16, torch.float16) or A.stride(1) != 1 or W.stride(1) != 1 or W.shape[0] != N:
        return None
    if out is None:
        out = torch.empty((M, N), dtype=A.dtype, device=A.device)
    if _C.RE_TUNE and M <= 128 and d == 128:
        from . import tuner
        tuner.maybe_tune(A.dtype, M, N, K, True, 2)
    cap = k_cache.shape[2] if k_cache is not None else 0
    rc = lib().kuiops_gemm_rope_qkv(dtype_code(A.dtype), M, hq, hk, d, K, A.data_ptr(), max(A.stride(0), K), W.data_ptr(), W.stride(0),
                                    out.data_ptr(), max(out.stride(0), N), positions.data_ptr(), float(theta), _ptr(k_cache),
                                    _ptr(v_cache), cap, rows_per_seq, _stream())
    if rc == EUNSUPPORTED:
        return None
    _check(rc, "gemm_rope_qkv")
    return out


def ssq_tiles(n):
    """Number of 128-feature tiles a row of n features is cut into by the folded-norm GEMMs."""
    return (int(n) + 127) // 128


def gemm_residual_ssq(A, W, resid, ssq):
    """resid += A @ W.T in place, and ssq[t, m] = sum of squares of tile t of row m as stored (the
    producer half of a folded RMSNorm).  Returns False when the shape does not suit the kernel."""
    M, K = A.shape
    N = W.shape[0]
    if (A.dtype not in (torch.bfloat16, torch.float16) or A.stride(1) != 1 or W.stride(1) != 1 or resid.stride(1) != 1
            or ssq.dtype != torch.float32 or ssq.numel() < ssq_tiles(N) * M or not ssq.is_contiguous()):
        return False
    rc = lib().kuiops_gemm_residual_ssq(dtype_code(A.dtype), M, N, K, A.data_ptr(), max(A.stride(0), K), W.data_ptr(), W.stride(0),
                                        resid.data_ptr(), max(resid.stride(0), N), ssq.data_ptr(), _stream())
    if rc == EUNSUPPORTED:
        return False
    _check(rc, "gemm_residual_ssq")
    return True


def gemm_swiglu_rms(A, W_interleaved, ssq, eps, out=None):
    """gemm_swiglu on un-normalised rows A, with row m scaled by rsqrt(sum_t ssq[t, m] / K + eps);
    None when the shape does not suit the kernel."""
    M, K = A.shape
    N = W_interleaved.shape[0] // 2
    if A.dtype not in (torch.bfloat16, torch.float16) or A.stride(1) != 1 or W_interleaved.stride(1) != 1:
        return None
    if out is None:
        out = torch.empty((M, N), dtype=A.dtype, device=A.device)
    rc = lib().kuiops_gemm_swiglu_rms(dtype_code(A.dtype), M, N, K, A.data_ptr(), max(A.stride(0), K), W_interleaved.data_ptr(),
                                      W_interleaved.stride(0), out.data_ptr(), max(out.stride(0), N), ssq.data_ptr(), ssq_tiles(K),
                                      float(eps), _stream())
    if rc == EUNSUPPORTED:
        return None
    _check(rc, "gemm_swiglu_rms")
    return out


def gemm_rope_qkv_rms(A, W, hq, hk, d, positions, theta, ssq, eps, k_cache=None, v_cache=None, rows_per_seq=1, out=None):
    """gemm_rope_qkv on un-normalised rows A, with row m scaled by rsqrt(sum_t ssq[t, m] / K + eps)."""
    M, K = A.shape
    N = (hq + 2 * hk) * d
    if A.dtype not in (torch.bfloat16, torch.float16) or A.stride(1) != 1 or W.stride(1) != 1 or W.shape[0] != N:
        return None
    if out is None:
        out = torch.empty((M, N), dtype=A.dtype, device=A.device)
    cap = k_cache.shape[2] if k_cache is not None else 0
    rc = lib().kuiops_gemm_rope_qkv_rms(dtype_code(A.dtype), M, hq, hk, d, K, A.data_ptr(), max(A.stride(0), K), W.data_ptr(), W.stride(0),
                                        out.data_ptr(), max(out.stride(0), N), positions.data_ptr(), float(theta), _ptr(k_cache),
                                        _ptr(v_cache), cap, rows_per_seq, ssq.data_ptr(), ssq_tiles(K), float(eps), _stream())
    if rc == EUNSUPPORTED:
        return None
    _check(rc, "gemm_rope_qkv_rms")
    return out


def gemm_push(A, B, *, trans_b, exchange):
    """Partial product of a row-split projection, stored into every rank's receive area of
    `exchange` (a kuillm_b200.peer.PeerExchange) instead of a local tensor."""
    M, K = A.shape
    N = B.shape[0] if trans_b else B.shape[1]
    x = exchange
    if M * N * 4 > x.slot_bytes:
        raise ValueError("kuiops: partial product larger than the exchange slots")
    _check(lib().kuiops_gemm_push(dtype_code(A.dtype), M, N, K, A.data_ptr(), max(A.stride(0), K), B.data_ptr(), B.stride(0),
                                  1 if trans_b else 0, x.n_ranks, x.rank, x.peer_array, x.slot_bytes,
                                  x.epoch.data_ptr(), _stream()), "gemm_push")


def rmsnorm_gather(exchange, rows, weight, eps, residual, out=None):
    """residual += sum of the ranks' partials; returns rmsnorm(residual) * weight (the consumer of gemm_push)."""
    x = exchange
    n = weight.shape[0]
    if residual.numel() != rows * n or not residual.is_contiguous() or rows * n * 4 > x.slot_bytes:
        raise ValueError("kuiops: rmsnorm_gather needs a contiguous [rows, n] residual that fits the exchange slots")
    if out is None:
        out = torch.empty((rows, n), dtype=weight.dtype, device=weight.device)
    _check(lib().kuiops_rmsnorm_gather(dtype_code(weight.dtype), rows, n, x.n_ranks, x.local_base, x.slot_bytes,
                                       x.epoch.data_ptr(), x.ticket_gather.data_ptr(), residual.data_ptr(), weight.data_ptr(),
                                       float(eps), out.data_ptr(), residual.data_ptr(), _stream()), "rmsnorm_gather")
    return out


def gemm_swiglu(A, W_interleaved, out=None):
    """silu(A Wg^T) * (A Wu^T) with gate / up rows interleaved in W ([2N, K]); falls back to the
    unfused pair of kernels where the tensor-core path does not apply."""
    M, K = A.shape
    N = W_interleaved.shape[0] // 2
    if out is None:
        out = torch.empty((M, N), dtype=A.dtype, device=A.device)
    L = lib()
    if _C.RE_TUNE and A.dtype in (torch.bfloat16, torch.float16):
        from . import tuner
        tuner.maybe_tune(A.dtype, M, 2 * N, K, True, 1)
    rc = L.kuiops_gemm_swiglu(dtype_code(A.dtype), M, N, K, A.data_ptr(), max(A.stride(0), K), W_interleaved.data_ptr(),
                              W_interleaved.stride(0), out.data_ptr(), max(out.stride(0), N), None, 0, _stream()) \
        if A.dtype in (torch.bfloat16, torch.float16) and A.stride(1) == 1 and W_interleaved.stride(1) == 1 else EUNSUPPORTED
    if rc == EUNSUPPORTED:
        gu = gemm(A, W_interleaved, trans_b=True)                      # interleaved columns
        g, u = gu[:, 0::2].contiguous(), gu[:, 1::2].contiguous()
        return swiglu(torch.cat([g, u], 1), out=out)
    _check(rc, "gemm_swiglu")
    return out


def mm(A, B):
    """aten.mm through the reference-order entry point (dense row-major operands)."""
    A, B = A.contiguous(), B.contiguous()
    M, K = A.shape
    N = B.shape[1]
    C = torch.empty((M, N), dtype=A.dtype, device=A.device)
    L = lib()
    ws = workspace("gemm", A.device, L.kuiops_gemm_workspace_bytes(dtype_code(A.dtype), 1, M, N, K))
    fn = getattr(L, f"kuiops_mm_{_sfx(A.dtype)}")
    _check(fn(M, N, K, A.data_ptr(), B.data_ptr(), C.data_ptr(), ws.data_ptr(), ws.numel(), _stream()), "mm")
    return C


def addmm(C, A, B, alpha, beta):
    """aten.addmm with a full [M,N] C, through the reference-order entry point (M, K, N)."""
    A, B = A.contiguous(), B.contiguous()
    out = C.contiguous().clone()
    M, K = A.shape
    N = B.shape[1]
    L = lib()
    ws = workspace("gemm", A.device, L.kuiops_gemm_workspace_bytes(dtype_code(A.dtype), 1, M, N, K))
    fn = getattr(L, f"kuiops_addmm_{_sfx(A.dtype)}")
    _check(fn(M, K, N, float(alpha), float(beta), A.data_ptr(), B.data_ptr(), out.data_ptr(),
              ws.data_ptr(), ws.numel(), _stream()), "addmm")
    return out


def bmm(A, B):
    A, B = A.contiguous(), B.contiguous()
    bsz, M, K = A.shape
    N = B.shape[2]
    C = torch.empty((bsz, M, N), dtype=A.dtype, device=A.device)
    L = lib()
    ws = workspace("gemm", A.device, L.kuiops_gemm_workspace_bytes(dtype_code(A.dtype), bsz, M, N, K))
    fn = getattr(L, f"kuiops_bmm_{_sfx(A.dtype)}")
    _check(fn(bsz, M, K, N, A.data_ptr(), B.data_ptr(), C.data_ptr(), ws.data_ptr(), ws.numel(), _stream()), "bmm")
    return C


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------
def sdpa(Q, K, V, *, bias=None, scale=None, is_causal=False, need_lse=True, out=None, kv_lens=None):
    """Q (n,h,l,e), K (n,h_kv,s,e), V (n,h_kv,s,ev) -> out (n,h,l,ev), lse (n,h,l) fp32.
    kv_lens: optional int64 device tensor [n] with the number of valid keys per batch entry."""
    n, h, l, e = Q.shape
    _, hkv, s, _ = K.shape
    ev = V.shape[3]
    if Q.stride(3) != 1:
        Q = Q.contiguous()
    if K.stride(3) != 1:
        K = K.contiguous()
    if V.stride(3) != 1:
        V = V.contiguous()
    if bias is not None:
        bias = bias.expand(n, h, l, s).contiguous()
    if scale is None:
        scale = 1.0 / (e ** 0.5)
    if out is None:
        out = torch.empty((n, h, l, ev), dtype=Q.dtype, device=Q.device)
    lse = torch.empty((n, h, l), dtype=torch.float32, device=Q.device) if need_lse else None
    L = lib()
    code = dtype_code(Q.dtype)
    wsb = L.kuiops_sdpa_workspace_bytes(code, n, h, hkv, l, s, e, ev)
    ws = workspace("sdpa", Q.device, wsb) if wsb else None
    args = (code, n, h, hkv, l, s, e, ev,
            Q.data_ptr(), Q.stride(0), Q.stride(1), Q.stride(2),
            K.data_ptr(), K.stride(0), K.stride(1), K.stride(2),
            V.data_ptr(), V.stride(0), V.stride(1), V.stride(2),
            _ptr(bias), float(scale), 1 if is_causal else 0,
            out.data_ptr(), out.stride(0), out.stride(1), out.stride(2), _ptr(lse))
    tail = (_ptr(ws), ws.numel() if ws is not None else 0, _stream())
    if kv_lens is None:
        _check(L.kuiops_sdpa(*args, *tail), "sdpa")
    else:
        _check(L.kuiops_sdpa_varlen(*args, kv_lens.data_ptr(), *tail), "sdpa_varlen")
    return out, lse


# --------------------------------------------------------------------------------------------
# streaming reductions
# --------------------------------------------------------------------------------------------
def softmax(X2d, out=None):
    """Row softmax of a contiguous [m, n] matrix; out may be X2d (in place)."""
    m, n = X2d.shape
    if out is None:
        out = torch.empty_like(X2d)
    fn = getattr(lib(), f"kuiops_softmax_{_sfx(X2d.dtype)}")
    _check(fn(m, n, X2d.data_ptr(), out.data_ptr(), _stream()), "softmax")
    return out


def mean_lastdim(X):
    Xc = X.contiguous()
    n = Xc.shape[-1]
    m = Xc.numel() // n
    out = torch.empty(tuple(Xc.shape[:-1]) + (1,), dtype=Xc.dtype, device=Xc.device)
    fn = getattr(lib(), f"kuiops_mean_{_sfx(Xc.dtype)}")
    _check(fn(m, n, Xc.data_ptr(), out.data_ptr(), _stream()), "mean")
    return out


def reduce(op, X):
    """Whole-tensor fold to a 0-d device tensor: op in {"all", "any", "max"}."""
    Xc = X.contiguous()
    code = dict(all=REDUCE_ALL, any=REDUCE_ANY, max=REDUCE_MAX)[op]
    if Xc.dtype in (torch.bool, torch.uint8):
        fn, odt = lib().kuiops_reduce_u8, Xc.dtype
    elif Xc.dtype == torch.int64:
        fn, odt = lib().kuiops_reduce_i64, torch.int64
    elif Xc.dtype == torch.float32:
        fn, odt = lib().kuiops_reduce_f32, torch.float32
    else:
        raise KuiopsError(EUNSUPPORTED, f"reduce over {Xc.dtype}")
    out = torch.empty((), dtype=odt, device=Xc.device)
    ws = workspace("reduce", Xc.device, REDUCE_WORKSPACE_BYTES)
    _check(fn(code, Xc.numel(), Xc.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), _stream()), "reduce")
    return out


def topk(X, k):
    """Largest-k over the last axis of fp32 X, sorted; equal values by ascending index."""
    Xc = X.contiguous()
    n = Xc.shape[-1]
    m = Xc.numel() // n
    vals = torch.empty(tuple(Xc.shape[:-1]) + (k,), dtype=torch.float32, device=Xc.device)
    idx = torch.empty(tuple(Xc.shape[:-1]) + (k,), dtype=torch.int64, device=Xc.device)
    _check(lib().kuiops_topk_f32(m, n, k, Xc.data_ptr(), vals.data_ptr(), idx.data_ptr(), _stream()), "topk")
    return vals, idx


def cast(X, dtype, out=None):
    """X converted to `dtype` (one of the float types); the same dtype gives a copy."""
    Xc = X.contiguous()
    if out is None:
        out = torch.empty(Xc.shape, dtype=dtype, device=Xc.device)
    if Xc.numel():
        _check(lib().kuiops_cast(dtype_code(Xc.dtype), dtype_code(dtype), Xc.numel(), Xc.data_ptr(), out.data_ptr(), _stream()), "cast")
    return out


def masked_fill(X, mask, value, out=None):
    Xc, Mc = X.contiguous(), mask.contiguous()
    if out is None:
        out = torch.empty_like(Xc)
    if Xc.numel():
        _check(lib().kuiops_masked_fill(dtype_code(Xc.dtype), Xc.numel(), Xc.data_ptr(), Mc.data_ptr(), float(value), out.data_ptr(),
                                        _stream()), "masked_fill")
    return out


def argmax_lastdim(X):
    Xc = X.contiguous()
    n = Xc.shape[-1]
    m = Xc.numel() // n
    out = torch.empty(tuple(Xc.shape[:-1]), dtype=torch.int64, device=Xc.device)
    _check(lib().kuiops_argmax(dtype_code(Xc.dtype), m, n, Xc.data_ptr(), out.data_ptr(), _stream()), "argmax")
    return out


def multinomial(P, num_samples=1, seed=0, offset=0):
    """One index per (row, sample) of the fp32 weight matrix P ([m, n] or [n]), drawn with replacement from the
    documented Philox stream (seed, offset); see kuiops_multinomial_f32."""
    if P.dtype != torch.float32:
        raise KuiopsError(EUNSUPPORTED, f"multinomial over {P.dtype}")
    Pc = P.contiguous()
    n = Pc.shape[-1]
    m = Pc.numel() // n
    out = torch.empty(tuple(Pc.shape[:-1]) + (num_samples,), dtype=torch.int64, device=Pc.device)
    _check(lib().kuiops_multinomial_f32(m, n, num_samples, Pc.data_ptr(), out.data_ptr(), int(seed) & (2 ** 64 - 1),
                                        int(offset) & (2 ** 64 - 1), _status(Pc.device).data_ptr(), _stream()), "multinomial")
    return out


def sample_topk_topp(logits, temperature=1.0, top_k=50, top_p=1.0, seed=0, offset=0, out=None, want_prob=False):
    """One token id per row of the fp32 logits ([m, n] or [n]): temperature, top-k, top-p and the draw from the
    documented Philox stream (seed, offset); see kuiops_sample_topk_topp_f32.  With want_prob also the picked
    token's probability under the filtered distribution."""
    if logits.dtype != torch.float32:
        raise KuiopsError(EUNSUPPORTED, f"sample over {logits.dtype}")
    Lc = logits.contiguous()
    n = Lc.shape[-1]
    m = Lc.numel() // n
    k = min(int(top_k), n)
    if out is None:
        out = torch.empty(tuple(Lc.shape[:-1]), dtype=torch.int64, device=Lc.device)
    prob = torch.empty(tuple(Lc.shape[:-1]), dtype=torch.float32, device=Lc.device) if want_prob else None
    nbytes = lib().kuiops_sample_workspace_bytes(m, max(k, 1))
    ws = workspace("sample", Lc.device, nbytes)
    _check(lib().kuiops_sample_topk_topp_f32(m, n, Lc.data_ptr(), float(temperature), int(top_k), float(top_p),
                                             int(seed) & (2 ** 64 - 1), int(offset) & (2 ** 64 - 1), out.data_ptr(), _ptr(prob),
                                             ws.data_ptr(), nbytes, _stream()), "sample_topk_topp")
    return (out, prob) if want_prob else out


def sort_lastdim(X, descending=False):
    """Stable sort of fp32 X over its last axis: (values, int64 indices)."""
    if X.dtype != torch.float32:
        raise KuiopsError(EUNSUPPORTED, f"sort over {X.dtype}")
    Xc = X.contiguous()
    n = Xc.shape[-1]
    m = Xc.numel() // n
    vals = torch.empty_like(Xc)
    idx = torch.empty(Xc.shape, dtype=torch.int64, device=Xc.device)
    nbytes = lib().kuiops_sort_workspace_bytes(m, n)
    ws = workspace("sort", Xc.device, nbytes)
    _check(lib().kuiops_sort_f32(m, n, 1 if descending else 0, Xc.data_ptr(), vals.data_ptr(), idx.data_ptr(),
                                 ws.data_ptr(), nbytes, _stream()), "sort")
    return vals, idx


def cumsum_lastdim(X, out=None):
    """Inclusive prefix sum over the last axis of a float32 or int64 tensor."""
    Xc = X.contiguous()
    n = Xc.shape[-1]
    m = Xc.numel() // n
    fn = {torch.float32: lib().kuiops_cumsum_f32, torch.int64: lib().kuiops_cumsum_i64}.get(Xc.dtype)
    if fn is None:
        raise KuiopsError(EUNSUPPORTED, f"cumsum over {Xc.dtype}")
    if out is None:
        out = torch.empty_like(Xc)
    elif out.shape != Xc.shape or out.dtype != Xc.dtype or not out.is_contiguous() or out.device != Xc.device:
        raise KuiopsError(EINVAL, "cumsum: out must be a dense tensor like the input")
    _check(fn(m, n, Xc.data_ptr(), out.data_ptr(), _stream()), "cumsum")
    return out


# --------------------------------------------------------------------------------------------
# indexed data movement
# --------------------------------------------------------------------------------------------
def _status(device):
    return workspace("status", device, 64)


def check_status(device):
    """Synchronising read of the out-of-range-index flag set by gather/scatter/index/embedding."""
    st = _status(device)
    flag = int(st[:4].view(torch.int32).item())
    if flag:
        st[:4].zero_()
    return flag


def gather(Inp, dim, Idx):
    Inp, Idx = Inp.contiguous(), Idx.contiguous()
    out = torch.empty(Idx.shape, dtype=Inp.dtype, device=Inp.device)
    _check(lib().kuiops_gather(Inp.element_size(), Inp.dim(), dim, _u64arr(Inp.shape), _u64arr(Idx.shape),
                               Inp.data_ptr(), Idx.data_ptr(), out.data_ptr(), Idx.numel(),
                               _status(Inp.device).data_ptr(), _stream()), "gather")
    return out


def scatter(Self, dim, Idx, Src):
    Self, Idx, Src = Self.contiguous(), Idx.contiguous(), Src.contiguous()
    out = torch.empty_like(Self)
    _check(lib().kuiops_scatter(Self.element_size(), Self.dim(), dim, _u64arr(Self.shape), _u64arr(Src.shape),
                                Self.data_ptr(), Src.data_ptr(), Idx.data_ptr(), out.data_ptr(), Src.numel(),
                                _status(Self.device).data_ptr(), _stream()), "scatter")
    return out


def cat2(A, B, dim):
    """Binary cat through the reference-order entry point."""
    A, B = A.contiguous(), B.contiguous()
    shape = list(A.shape)
    shape[dim] = A.shape[dim] + B.shape[dim]
    out = torch.empty(shape, dtype=A.dtype, device=A.device)
    _check(lib().kuiops_cat(A.element_size(), A.dim(), dim, _u64arr(A.shape), B.shape[dim],
                            A.data_ptr(), B.data_ptr(), out.data_ptr(), out.numel(), _stream()), "cat")
    return out


def cat(tensors, dim):
    tensors = [t.contiguous() for t in tensors]
    shape = list(tensors[0].shape)
    sizes = [t.shape[dim] for t in tensors]
    shape[dim] = sum(sizes)
    out = torch.empty(shape, dtype=tensors[0].dtype, device=tensors[0].device)
    ptrs = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    _check(lib().kuiops_cat_n(out.element_size(), out.dim(), dim, len(tensors), _u64arr(tensors[0].shape),
                              _u64arr(sizes), ptrs, out.data_ptr(), _stream()), "cat_n")
    return out


def index(Self, first_dim, indices):
    """Self[..., i0, i1, ..., ...] with int64 index tensors on adjacent dims starting at first_dim."""
    Self = Self.contiguous()
    bshape = torch.broadcast_shapes(*[i.shape for i in indices])
    exp = [i.expand(bshape) for i in indices]     # views: broadcast dims get stride 0
    keep = []                                     # the expanded views must stay dense elsewhere
    strides = []
    for v, orig in zip(exp, indices):
        if not orig.is_contiguous():
            orig = orig.contiguous()
            v = orig.expand(bshape)
        keep.append(orig)
        strides += list(v.stride())
    out_shape = tuple(Self.shape[:first_dim]) + tuple(bshape) + tuple(Self.shape[first_dim + len(indices):])
    out = torch.empty(out_shape, dtype=Self.dtype, device=Self.device)
    if out.numel() == 0:
        return out
    ptrs = (ctypes.c_void_p * len(indices))(*[k.data_ptr() for k in keep])
    stride_arr = (ctypes.c_int64 * max(1, len(strides)))(*strides)
    _check(lib().kuiops_index(Self.element_size(), Self.dim(), _u64arr(Self.shape), first_dim, len(indices), ptrs,
                              len(bshape), _u64arr(bshape) if len(bshape) else None, stride_arr,
                              Self.data_ptr(), out.data_ptr(), _status(Self.device).data_ptr(), _stream()), "index")
    return out


def isin(elements, test_elements, invert=False):
    e, t = elements.contiguous(), test_elements.contiguous().reshape(-1)
    out = torch.empty(e.shape, dtype=torch.bool, device=e.device)
    if e.numel() == 0:
        return out
    _check(lib().kuiops_isin_i64(e.numel(), e.data_ptr(), t.numel(), _ptr(t) if t.numel() else None,
                                 1 if invert else 0, out.data_ptr(), _stream()), "isin")
    return out


# --------------------------------------------------------------------------------------------
# elementwise maps
# --------------------------------------------------------------------------------------------
def map1(op, X, c0=0.0, c1=1.0, out=None):
    Xc = X.contiguous()
    if out is None:
        out = torch.empty_like(Xc)
    _check(lib().kuiops_map(dtype_code(Xc.dtype), MAP[op], Xc.numel(), Xc.data_ptr(), out.data_ptr(),
                            float(c0), float(c1), _stream()), f"map {op}")
    return out


def add_i64_(x, delta):
    """In-place x += delta on an int64 device tensor."""
    _check(lib().kuiops_add_i64(x.numel(), x.data_ptr(), int(delta), _stream()), "add_i64")
    return x


def map2(op, X, B, c1=1.0, out=None):
    Xc, Bc = X.contiguous(), B.contiguous()
    if out is None:
        out = torch.empty_like(Xc)
    _check(lib().kuiops_map2(dtype_code(Xc.dtype), MAP[op], Xc.numel(), Xc.data_ptr(), Bc.data_ptr(),
                             out.data_ptr(), float(c1), _stream()), f"map2 {op}")
    return out


def map_u8(op, X, B=None):
    Xc = X.contiguous()
    Bc = B.contiguous() if B is not None else None
    out = torch.empty_like(Xc)
    _check(lib().kuiops_map_u8(MAP[op], Xc.numel(), Xc.data_ptr(), _ptr(Bc), out.data_ptr(), _stream()), f"map_u8 {op}")
    return out


def map_nip(op, X, c0):
    Xc = X.contiguous()
    out = torch.empty(Xc.shape, dtype=torch.bool, device=Xc.device)
    _check(lib().kuiops_map_nip(dtype_code(Xc.dtype), MAP[op], Xc.numel(), Xc.data_ptr(), out.data_ptr(),
                                float(c0), _stream()), f"map_nip {op}")
    return out


def where(cond, A, B):
    c, a, b = cond.contiguous(), A.contiguous(), B.contiguous()
    out = torch.empty_like(a)
    _check(lib().kuiops_map3(a.element_size(), a.numel(), c.data_ptr(), a.data_ptr(), b.data_ptr(),
                             out.data_ptr(), _stream()), "where")
    return out


# --------------------------------------------------------------------------------------------
# fused decoder-layer helpers
# --------------------------------------------------------------------------------------------
def rmsnorm(x, weight, eps, residual=None, out=None, residual_out=None):
    n = x.shape[-1]
    m = x.numel() // n
    if out is None:
        out = torch.empty_like(x)
    if residual is not None and residual_out is None:
        residual_out = residual
    _check(lib().kuiops_rmsnorm(dtype_code(x.dtype), m, n, x.data_ptr(), _ptr(residual), weight.data_ptr(),
                                float(eps), out.data_ptr(), _ptr(residual_out), _stream()), "rmsnorm")
    return out


def swiglu(gate_up, out=None):
    n2 = gate_up.shape[-1]
    m = gate_up.numel() // n2
    if out is None:
        out = torch.empty(tuple(gate_up.shape[:-1]) + (n2 // 2,), dtype=gate_up.dtype, device=gate_up.device)
    _check(lib().kuiops_swiglu(dtype_code(gate_up.dtype), m, n2 // 2, gate_up.data_ptr(), out.data_ptr(),
                               _stream()), "swiglu")
    return out


def rope_qkv(qkv, hq, hk, d, positions, theta, k_cache=None, v_cache=None, rows_per_seq=1):
    rows = qkv.numel() // qkv.shape[-1]
    cap = k_cache.shape[2] if k_cache is not None else 0
    _check(lib().kuiops_rope_qkv(dtype_code(qkv.dtype), rows, hq, hk, d, qkv.data_ptr(), qkv.stride(-2) if qkv.dim() > 1 else qkv.shape[-1],
                                 positions.data_ptr(), float(theta), _ptr(k_cache), _ptr(v_cache), cap,
                                 rows_per_seq, _stream()), "rope_qkv")
    return qkv


def embedding(table, ids):
    ids_c = ids.contiguous()
    out = torch.empty(tuple(ids_c.shape) + (table.shape[1],), dtype=table.dtype, device=table.device)
    _check(lib().kuiops_embedding(table.element_size(), ids_c.numel(), table.shape[1], table.shape[0],
                                  table.data_ptr(), ids_c.data_ptr(), out.data_ptr(),
                                  _status(table.device).data_ptr(), _stream()), "embedding")
    return out
