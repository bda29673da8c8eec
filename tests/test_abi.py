"""The C ABI: the library loads without a GPU, exports every symbol ``include/kuiops.h``
declares, the ctypes table binds each of them, and contract violations are refused on the host
(nothing is launched, so these run on CPU).  The contracts are the F* refinements of the
reference (Kuiops.Common.fsti:34-38 shape_le; Kuiops.Gather.fsti:31-33; Kuiops.Cat.fsti:50-52;
Kuiops.Mean.fsti:41-42) turned into runtime checks."""
import ctypes
import re
from pathlib import Path

import pytest

from kuipy import _ffi

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "kuiops.h").read_text()
DECLARED = re.findall(r"KUIOPS_API\s+[\w\s\*]+?\b(kuiops_\w+)\s*\(", HEADER)
P = 0x1000   # a non-null pointer that is never dereferenced: every call below fails its checks first


def u64(*v):
    return (ctypes.c_uint64 * len(v))(*v)


def test_header_declares_the_expected_surface():
    assert len(DECLARED) == len(set(DECLARED)) >= 40
    for must in ("kuiops_mm_bf16", "kuiops_addmm_f32", "kuiops_bmm_f16", "kuiops_gemm", "kuiops_sdpa",
                 "kuiops_softmax_f32", "kuiops_mean_bf16", "kuiops_topk_f32", "kuiops_gather", "kuiops_scatter",
                 "kuiops_cat", "kuiops_cat_n", "kuiops_index", "kuiops_isin_i64", "kuiops_map", "kuiops_reduce_u8"):
        assert must in DECLARED


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_ffi.LIB_PATH))
    missing = [n for n in DECLARED if not hasattr(lib, n)]
    assert not missing, missing


def test_ctypes_table_covers_the_header():
    assert set(_ffi.SIGNATURES) == set(DECLARED)
    assert _ffi.lib().kuiops_abi_version() == 1
    assert "contract" in _ffi.strerror(_ffi.EINVAL)


def test_every_declaration_cites_the_reference_or_says_it_has_no_counterpart():
    # each entry-point comment names the reference launcher (a .j2 / .fst / .md path) it replaces
    blocks = re.split(r"\n\s*\n", HEADER)
    for b in blocks:
        names = re.findall(r"KUIOPS_API[^;]*?\b(kuiops_(?:mm|addmm|bmm|softmax|mean|gather|scatter|cat|index|isin|topk|sdpa|map|reduce)\w*)\s*\(", b)
        if names:
            assert re.search(r"\.j2|\.fst|KERNELS\.md|kuipy/|No reference|[Nn]o counterpart", b), names


def test_gemm_contracts():
    L = _ffi.lib()
    f = L.kuiops_gemm
    ok_tail = (P, 64, 0, P, 64, 0, 0, None, 0, 0, 1.0, 0.0, P, 64, 0, None, 0, None)
    assert f(_ffi.F32, _ffi.F32, 1, 0, 64, 64, *ok_tail) == _ffi.EINVAL            # M == 0
    assert f(7, 7, 1, 64, 64, 64, *ok_tail) == _ffi.EINVAL                          # unknown dtype
    assert f(_ffi.F32, _ffi.BF16, 1, 64, 64, 64, *ok_tail) == _ffi.EINVAL           # out dtype must be in dtype or f32
    assert f(_ffi.F32, _ffi.F32, 1, 64, 64, 64, None, 64, 0, P, 64, 0, 0, None, 0, 0, 1.0, 0.0, P, 64, 0, None, 0, None) == _ffi.EINVAL
    assert f(_ffi.F32, _ffi.F32, 1, 64, 64, 64, P, 32, 0, P, 64, 0, 0, None, 0, 0, 1.0, 0.0, P, 64, 0, None, 0, None) == _ffi.EINVAL  # lda < K
    # split-K partials live in shared memory (cluster reduction): no shape needs more than the fixed head
    assert L.kuiops_gemm_workspace_bytes(_ffi.BF16, 1, 16, 4096, 4096) == _ffi.GEMM_COUNTER_BYTES
    assert L.kuiops_gemm_workspace_bytes(_ffi.BF16, 1, 4096, 4096, 4096) == _ffi.GEMM_COUNTER_BYTES


def test_tensor_parallel_push_and_gather_contracts():
    """Argument checks of the fused all-reduce pair; nothing is launched (no GPU here)."""
    import ctypes
    L = _ffi.lib()
    peers = (ctypes.c_uint64 * 2)(0x1000, 0x2000)
    slot = 32 * 4096 * 4                                                 # 4 bytes per element: value + half a stamp
    ok = dict(M=32, N=4096, K=2048)

    def push(dtype=_ffi.BF16, M=32, N=4096, n_ranks=2, rank=0, peer_array=peers, slot_bytes=slot, epoch=P):
        return L.kuiops_gemm_push(dtype, M, N, ok["K"], P, ok["K"], P, ok["K"], 1, n_ranks, rank, peer_array,
                                  slot_bytes, epoch, None)
    assert push(dtype=_ffi.F32) == _ffi.EUNSUPPORTED                     # 16-bit operands only
    assert push(M=256) == _ffi.EUNSUPPORTED                              # decode-sized steps only
    assert push(N=4098, slot_bytes=32 * 4098 * 4) == _ffi.EUNSUPPORTED   # cells hold element pairs, stored two at a time
    assert push(n_ranks=1) == _ffi.EINVAL and push(n_ranks=9) == _ffi.EINVAL and push(rank=2) == _ffi.EINVAL
    assert push(slot_bytes=slot - 16) == _ffi.EINVAL                     # a slot must hold the M x N partial with its stamps
    assert push(slot_bytes=32 * 4096 * 2) == _ffi.EINVAL                 # ... which is twice the bytes of the bare elements
    assert push(peer_array=(ctypes.c_uint64 * 2)(0x1000, 0)) == _ffi.EINVAL
    assert push(peer_array=(ctypes.c_uint64 * 2)(0x1000, 0x2008)) == _ffi.EINVAL     # 16-byte alignment
    assert push(epoch=None) == _ffi.EINVAL

    def gather(dtype=_ffi.BF16, m=32, n=4096, n_ranks=2, slot_bytes=slot, residual=P):
        return L.kuiops_rmsnorm_gather(dtype, m, n, n_ranks, P, slot_bytes, P, P, residual, P, 1e-5, P, P, None)
    assert gather(dtype=_ffi.F32) == _ffi.EUNSUPPORTED
    assert gather(m=0) == _ffi.EINVAL and gather(n_ranks=1) == _ffi.EINVAL and gather(residual=None) == _ffi.EINVAL
    assert gather(slot_bytes=slot - 16) == _ffi.EINVAL
    assert gather(n=4100, slot_bytes=32 * 4100 * 4) == _ffi.EUNSUPPORTED   # rows must be whole 16-byte vectors


def test_qkv_projection_with_rope_epilogue_contracts():
    """Argument checks of the fused QKV projection; every call below is refused before a launch."""
    L = _ffi.lib()

    def qkv(dtype=_ffi.BF16, M=32, hq=32, hk=8, d=128, K=4096, lda=4096, ldw=4096, ldq=48 * 128, positions=P,
            theta=5e5, k_cache=P, v_cache=P, cap=4096):
        return L.kuiops_gemm_rope_qkv(dtype, M, hq, hk, d, K, P, lda, P, ldw, P, ldq, positions, theta,
                                      k_cache, v_cache, cap, 1, None)
    assert qkv(dtype=_ffi.F32) == _ffi.EUNSUPPORTED                      # 16-bit operands only
    assert qkv(M=0) == _ffi.EINVAL and qkv(positions=None) == _ffi.EINVAL and qkv(theta=0.0) == _ffi.EINVAL
    assert qkv(v_cache=None) == _ffi.EINVAL                              # both caches or neither
    assert qkv(cap=0) == _ffi.EINVAL                                     # a cache needs a capacity
    assert qkv(d=64) == _ffi.EUNSUPPORTED and qkv(M=256) == _ffi.EUNSUPPORTED
    assert qkv(ldq=47 * 128) == _ffi.EINVAL and qkv(lda=2048) == _ffi.EINVAL and qkv(ldw=2048) == _ffi.EINVAL


def test_softmax_mean_topk_contracts():
    L = _ffi.lib()
    assert L.kuiops_softmax_f32(0, 8, P, P, None) == _ffi.EINVAL
    assert L.kuiops_softmax_f32(8, 8, None, P, None) == _ffi.EINVAL
    assert L.kuiops_mean_bf16(4, 0, P, P, None) == _ffi.EINVAL
    assert L.kuiops_topk_f32(4, 10, 11, P, P, P, None) == _ffi.EINVAL                # k > n
    assert L.kuiops_topk_f32(4, 100000, 4096, P, P, P, None) == _ffi.ELIMIT          # k beyond the fixed maximum
    assert L.kuiops_reduce_u8(_ffi.REDUCE_ALL, 16, P, P, None, 0, None) == _ffi.EWORKSPACE
    assert L.kuiops_reduce_i64(_ffi.REDUCE_ALL, 16, P, P, P, 1 << 20, None) == _ffi.EUNSUPPORTED


def test_cumsum_contracts():
    L = _ffi.lib()
    for f in (L.kuiops_cumsum_f32, L.kuiops_cumsum_i64):
        assert f(0, 8, P, P, None) == _ffi.EINVAL and f(8, 0, P, P, None) == _ffi.EINVAL
        assert f(8, 8, None, P, None) == _ffi.EINVAL and f(8, 8, P, None, None) == _ffi.EINVAL
        assert f(1 << 16, (1 << 15) + 1, P, P, None) == _ffi.ELIMIT          # m * n <= 2^31


def test_sort_contracts():
    L = _ffi.lib()
    assert L.kuiops_sort_workspace_bytes(64, 128256) == 64 * 128256 * 16
    f = L.kuiops_sort_f32
    big = 1 << 30
    assert f(0, 8, 0, P, P + big, P, P, 1 << 20, None) == _ffi.EINVAL and f(8, 8, 0, None, P, P, P, 1 << 20, None) == _ffi.EINVAL
    assert f(8, 8, 0, P, P + big, P, None, 0, None) == _ffi.EWORKSPACE
    assert f(8, 8, 0, P, P + big, P, P, 8 * 8 * 16 - 1, None) == _ffi.EWORKSPACE
    assert f(8, 8, 0, P, P + 64, P, P, 1 << 20, None) == _ffi.EINVAL           # values overlap the input
    assert f(1 << 16, (1 << 15) + 1, 0, P, P + (1 << 40), P, P, 1 << 62, None) == _ffi.ELIMIT


def test_gather_scatter_contracts():
    L = _ffi.lib()
    # shape_le off the gathered axis
    assert L.kuiops_gather(4, 2, 1, u64(4, 4), u64(5, 4), P, P, P, 20, None, None) == _ffi.EINVAL
    # n must equal numel(idx)
    assert L.kuiops_gather(4, 2, 1, u64(4, 4), u64(4, 3), P, P, P, 11, None, None) == _ffi.EINVAL
    # element size, rank, dim
    assert L.kuiops_gather(3, 2, 1, u64(4, 4), u64(4, 4), P, P, P, 16, None, None) == _ffi.EINVAL
    assert L.kuiops_gather(4, 9, 1, u64(*[2] * 9), u64(*[2] * 9), P, P, P, 512, None, None) == _ffi.EINVAL
    assert L.kuiops_gather(4, 2, 2, u64(4, 4), u64(4, 4), P, P, P, 16, None, None) == _ffi.EINVAL
    # empty index
    assert L.kuiops_gather(4, 2, 1, u64(4, 4), u64(0, 4), P, P, P, 0, None, None) == _ffi.EINVAL
    assert L.kuiops_scatter(4, 2, 1, u64(4, 4), u64(4, 5), P, P, P, P, 20, None, None) == _ffi.EINVAL
    assert L.kuiops_scatter(4, 2, 1, u64(4, 4), u64(4, 4), P, P, P, P, 15, None, None) == _ffi.EINVAL


def test_cat_index_isin_contracts():
    L = _ffi.lib()
    # out_dim = a_dim + b_dim
    assert L.kuiops_cat(4, 2, 1, u64(4, 4), 2, P, P, P, 4 * 7, None) == _ffi.EINVAL
    assert L.kuiops_cat(4, 2, 3, u64(4, 4), 2, P, P, P, 24, None) == _ffi.EINVAL
    ptrs = (ctypes.c_void_p * 2)(P, P)
    assert L.kuiops_cat_n(4, 2, 1, 0, u64(4, 4), u64(4, 4), ptrs, P, None) == _ffi.EINVAL
    assert L.kuiops_index(4, 2, u64(4, 4), 1, 2, ptrs, 1, u64(3), (ctypes.c_int64 * 2)(1, 1), P, P, None, None) == _ffi.EINVAL
    assert L.kuiops_isin_i64(0, P, 4, P, 0, P, None) == _ffi.EINVAL


def test_sdpa_contracts():
    L = _ffi.lib()
    base = [_ffi.BF16, 2, 8, 3, 4, 16, 128, 128]                # h = 8 not a multiple of h_kv = 3
    tail = [P, 1, 1, 128, P, 1, 1, 128, P, 1, 1, 128, None, 1.0, 1, P, 1, 1, 128, None, None, 0, None]
    assert L.kuiops_sdpa(*base, *tail) == _ffi.EINVAL
    base[3] = 2
    bad = list(tail)
    bad[3] = 64                                                  # q row stride < e
    assert L.kuiops_sdpa(*base, *bad) == _ffi.EINVAL
    assert L.kuiops_sdpa_workspace_bytes(_ffi.BF16, 64, 32, 8, 1, 32768, 128, 128) == 0   # enough (batch, kv head) units: no split
    assert L.kuiops_sdpa_workspace_bytes(_ffi.BF16, 1, 32, 8, 1, 32768, 128, 128) > 0     # one sequence: keys are split
