"""``kuiops_sdpa_noalloc``: attention for hosts that cannot allocate device memory (a plugin
inside a runtime that owns the whole device pool; a serving loop that cannot take an allocation
stall).  Its split-KV scratch is a fixed array inside the library instead of a caller buffer.

Called through the C ABI and compared with ``kuiops_sdpa`` (caller-provided scratch) on the same
inputs, twice in a row with different data, because every call reuses the one array and finds
the previous call's contents in it.  Collected last on purpose."""
import ctypes

import pytest
import torch

from kuipy import _ffi

pytestmark = pytest.mark.gpu


def _call_noalloc(Q, K, V, causal, kv_lens=None):
    n, h, l, e = Q.shape
    hkv, s, ev = K.shape[1], K.shape[2], V.shape[3]
    out = torch.empty((n, h, l, ev), dtype=Q.dtype, device=Q.device)
    lse = torch.empty((n, h, l), dtype=torch.float32, device=Q.device)
    rc = _ffi.lib().kuiops_sdpa_noalloc(
        _ffi.dtype_code(Q.dtype), n, h, hkv, l, s, e, ev,
        Q.data_ptr(), Q.stride(0), Q.stride(1), Q.stride(2),
        K.data_ptr(), K.stride(0), K.stride(1), K.stride(2),
        V.data_ptr(), V.stride(0), V.stride(1), V.stride(2),
        None, 1.0 / e ** 0.5, 1 if causal else 0,
        out.data_ptr(), out.stride(0), out.stride(1), out.stride(2), lse.data_ptr(),
        None if kv_lens is None else kv_lens.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == _ffi.OK, _ffi.strerror(rc)
    return out, lse


def _max_rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-30)).item()


def test_noalloc_matches_the_caller_scratch_entry_point_twice(cuda):
    shape = dict(n=2, h=32, hkv=8, s=8192)             # few (batch, kv head) units: the keys are split over CTAs
    need = _ffi.lib().kuiops_sdpa_workspace_bytes(_ffi.BF16, shape["n"], shape["h"], shape["hkv"], 1, shape["s"], 128, 128)
    assert 0 < need <= _ffi.SDPA_NOALLOC_SCRATCH_BYTES, "the case must exercise the scratch path"
    for seed in (0, 1):                                # second call meets the first call's leftovers
        g = torch.Generator(device="cuda").manual_seed(seed)
        Q = torch.randn(shape["n"], shape["h"], 1, 128, device="cuda", generator=g).bfloat16()
        K = torch.randn(shape["n"], shape["hkv"], shape["s"], 128, device="cuda", generator=g).bfloat16()
        V = torch.randn(shape["n"], shape["hkv"], shape["s"], 128, device="cuda", generator=g).bfloat16()
        ref_out, ref_lse = _ffi.sdpa(Q, K, V, is_causal=True)
        out, lse = _call_noalloc(Q, K, V, True)
        torch.cuda.synchronize()
        assert _max_rel(out, ref_out) <= 2e-2 and _max_rel(lse, ref_lse) <= 2e-2
        lens = torch.tensor([5000, 8192], device="cuda")
        ref_out, _ = _ffi.sdpa(Q, K, V, is_causal=True, kv_lens=lens)
        out, _ = _call_noalloc(Q, K, V, True, kv_lens=lens)
        torch.cuda.synchronize()
        assert _max_rel(out, ref_out) <= 2e-2


def test_noalloc_alternating_kernels_share_the_array(cuda):
    """The two split-KV kernels lay out different ticket blocks at the head of the one array: an
    fp32 call (SIMT rows kernel) and a bf16 call (tensor-core decode kernel) follow each other in
    both orders, each finding the other's records, and each must agree with ``kuiops_sdpa``."""
    def case(dtype, seed):
        g = torch.Generator(device="cuda").manual_seed(seed)
        mk = lambda *shape: torch.randn(*shape, device="cuda", generator=g).to(dtype)
        return mk(1, 8, 1, 128), mk(1, 2, 6000, 128), mk(1, 2, 6000, 128)
    order = [(torch.bfloat16, 0), (torch.float32, 1), (torch.bfloat16, 2), (torch.float32, 3), (torch.float32, 4), (torch.bfloat16, 5)]
    for dtype, seed in order:
        Q, K, V = case(dtype, seed)
        code = _ffi.dtype_code(dtype)
        assert _ffi.lib().kuiops_sdpa_workspace_bytes(code, 1, 8, 2, 1, 6000, 128, 128) > 0, "must be a split-KV case"
        ref_out, ref_lse = _ffi.sdpa(Q, K, V, is_causal=True)
        out, lse = _call_noalloc(Q, K, V, True)
        torch.cuda.synchronize()
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
        assert _max_rel(out, ref_out) <= tol and _max_rel(lse, ref_lse) <= tol, (dtype, seed)


def test_noalloc_uses_the_array_of_the_gpu_that_holds_the_inputs(cuda):
    """With two GPUs visible: inputs on GPU 1 while GPU 0 is the calling thread's current device,
    after GPU 0 has already been used.  The entry point has to pick GPU 1's copy of the array."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    g = torch.Generator().manual_seed(9)
    Q, K, V = (torch.randn(s, generator=g).bfloat16() for s in ((2, 32, 1, 128), (2, 8, 8192, 128), (2, 8, 8192, 128)))
    outs = []
    for dev in (0, 1):
        q, k, v = Q.to(f"cuda:{dev}"), K.to(f"cuda:{dev}"), V.to(f"cuda:{dev}")
        with torch.cuda.device(dev):
            ref, _ = _ffi.sdpa(q, k, v, is_causal=True)
        torch.cuda.set_device(0)                        # current device stays GPU 0 for the call itself
        out = torch.empty_like(ref)
        rc = _ffi.lib().kuiops_sdpa_noalloc(
            _ffi.BF16, 2, 32, 8, 1, 8192, 128, 128,
            q.data_ptr(), q.stride(0), q.stride(1), q.stride(2), k.data_ptr(), k.stride(0), k.stride(1), k.stride(2),
            v.data_ptr(), v.stride(0), v.stride(1), v.stride(2), None, 1.0 / 128 ** 0.5, 1,
            out.data_ptr(), out.stride(0), out.stride(1), out.stride(2), None, None,
            torch.cuda.current_stream(dev).cuda_stream)
        assert rc == _ffi.OK, _ffi.strerror(rc)
        torch.cuda.synchronize(dev)
        assert _max_rel(out, ref) <= 2e-2
        outs.append(out.cpu())
    assert torch.equal(outs[0], outs[1])


def test_noalloc_refuses_problems_beyond_its_fixed_scratch(cuda):
    # 295 kv heads x 16 query heads each: the split-KV records need more than the built-in array
    n, hkv, g, s = 1, 295, 16, 4096
    need = _ffi.lib().kuiops_sdpa_workspace_bytes(_ffi.BF16, n, hkv * g, hkv, 1, s, 128, 256)
    assert need > _ffi.SDPA_NOALLOC_SCRATCH_BYTES
    P = 0x1000                                          # never dereferenced: the size check comes first
    rc = _ffi.lib().kuiops_sdpa_noalloc(_ffi.BF16, n, hkv * g, hkv, 1, s, 128, 256,
                                        P, 128, 128, 128, P, 128, 128, 128, P, 256, 256, 256,
                                        None, 1.0, 1, P, 256, 256, 256, None, None, None)
    assert rc == _ffi.ELIMIT and "maximum" in _ffi.strerror(rc)
