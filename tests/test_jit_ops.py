"""Per-family parity on a GPU: ``impl.supported()`` then ``impl.run()`` (which calls the C ABI),
checked against the CPU oracle on seeded inputs.  Shapes and tolerances follow the reference's
tests/test_jit_ops.py; the attention tests it keeps skipped run here, and the new families
(topk, isin, index, reduce, n-ary cat, 1-D bias) are added."""
import numpy as np
import pytest
import torch

from kuipy import kuiops
from oracle import kuiops_oracle as O
from _util import (assert_bit_exact, assert_close_ref_bar, assert_fp32_1e5, assert_max_rel, run_family, to_np)

pytestmark = pytest.mark.gpu
aten = torch.ops.aten
FLOATS = [torch.float32, torch.bfloat16, torch.float16]


def randn(*shape, dtype=torch.float32, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype).cuda()


# ---- GEMM family ------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", FLOATS)
def test_bmm(cuda, dtype):
    A, B = randn(5, 17, 9, dtype=dtype), randn(5, 9, 13, dtype=dtype, seed=1)
    out = run_family(kuiops.BmmImpl({}), aten.bmm.default, (A, B))
    assert out.dtype == dtype
    assert_close_ref_bar(out, O.bmm(to_np(A), to_np(B)), dtype)


def test_bmm_unsupported(cuda):
    impl = kuiops.BmmImpl({})
    assert impl.supported(aten.bmm.default, (randn(2, 4, 4), randn(3, 4, 4)), {}) is None
    assert impl.supported(aten.bmm.default, (randn(4, 4), randn(4, 4)), {}) is None


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("alpha,beta", [(1.0, 1.0), (0.5, 2.0)])
def test_addmm_full_matrix(cuda, dtype, alpha, beta):
    M = K = N = 64
    A, B, Cm = randn(M, K, dtype=dtype), randn(K, N, dtype=dtype, seed=1), randn(M, N, dtype=dtype, seed=2)
    out = run_family(kuiops.AddmmImpl({}), aten.addmm.default, (Cm, A, B), dict(alpha=alpha, beta=beta))
    assert_close_ref_bar(out, O.addmm(to_np(Cm), to_np(A), to_np(B), alpha, beta), dtype)
    assert Cm.data_ptr() != out.data_ptr()


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("alpha,beta", [(1.0, 1.0), (0.5, 2.0)])
def test_addmm_1d_bias(cuda, gates, dtype, alpha, beta):
    gates("wide")
    M, K, N = 64, 64, 64
    A, B, bias = randn(M, K, dtype=dtype), randn(K, N, dtype=dtype, seed=1), randn(N, dtype=dtype, seed=2)
    out = run_family(kuiops.AddmmImpl({}), aten.addmm.default, (bias, A, B), dict(alpha=alpha, beta=beta))
    assert_close_ref_bar(out, O.addmm(to_np(bias), to_np(A), to_np(B), alpha, beta), dtype)


def test_addmm_rejections(cuda, gates):
    gates("reference")
    impl = kuiops.AddmmImpl({})
    d = lambda *s: torch.randn(*s, device="cuda", dtype=torch.float64)
    assert impl.supported(aten.addmm.default, (d(32, 32), d(32, 32), d(32, 32)), {}) is None
    A, B = randn(32, 32), randn(32, 32)
    assert impl.supported(aten.addmm.default, (randn(32), A, B), {}) is None
    assert impl.supported(aten.addmm.default, (randn(1, 32), A, B), {}) is None


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("shape", [(64, 64, 64), (128, 128, 64), (17, 13, 9), (1, 40, 24), (130, 72, 200), (16, 256, 512)])
def test_mm_shapes(cuda, gates, dtype, shape):
    gates("wide")
    M, N, K = shape
    A, B = randn(M, K, dtype=dtype), (randn(K, N, dtype=dtype, seed=1) / K ** 0.5).to(dtype)
    out = run_family(kuiops.MmImpl({}), aten.mm.default, (A, B))
    assert out.dtype == dtype and tuple(out.shape) == (M, N)
    assert_close_ref_bar(out, O.mm(to_np(A), to_np(B)), dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_mm_transposed_weight_view_is_used_in_place(cuda, gates, dtype):
    gates("wide")
    W, A = randn(96, 128, dtype=dtype, seed=3), randn(24, 128, dtype=dtype)      # Linear: A @ W.t()
    out = run_family(kuiops.MmImpl({}), aten.mm.default, (A, W.t()))
    assert_close_ref_bar(out, O.mm(to_np(A), to_np(W).T), dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M", [1, 7, 32, 100, 300])
def test_gemm_swiglu_fused_epilogue(cuda, dtype, M):
    from kuipy import _ffi
    N, K = 200, 136
    A = randn(M, K, dtype=dtype)
    Wg, Wu = (randn(N, K, dtype=dtype, seed=1) / K ** 0.5).to(dtype), (randn(N, K, dtype=dtype, seed=2) / K ** 0.5).to(dtype)
    W = torch.stack([Wg, Wu], 1).reshape(2 * N, K).contiguous()
    out = _ffi.gemm_swiglu(A, W)
    g, u = O.mm(to_np(A), to_np(Wg).T), O.mm(to_np(A), to_np(Wu).T)
    ref = g / (1.0 + np.exp(-g)) * u
    assert out.shape == (M, N) and out.dtype == dtype
    assert_close_ref_bar(out, ref, dtype)
    assert _ffi.tc_error() == 0


def test_mm_many_row_tiles_walked_in_bands(cuda):
    """More than 32 row tiles with a ragged last band and a ragged last tile: every output tile is
    produced exactly once whatever order the tiles are walked in."""
    from kuipy import _ffi
    A, B = randn(4700, 192, dtype=torch.bfloat16), randn(520, 192, dtype=torch.bfloat16, seed=1)
    out = _ffi.gemm(A, B, trans_b=True)
    assert_close_ref_bar(out, O.mm(to_np(A), to_np(B).T), torch.bfloat16)
    bias = randn(520, dtype=torch.bfloat16, seed=2)
    out = _ffi.gemm(A, B, trans_b=True, Cin=bias)
    assert_close_ref_bar(out, O.mm(to_np(A), to_np(B).T) + to_np(bias)[None, :], torch.bfloat16)
    assert _ffi.tc_error() == 0


# ---- softmax / mean / folds / topk -----------------------------------------------------------------
@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("shape", [(128, 64), (8, 5, 33), (3, 4100), (2, 40000)])
def test_softmax(cuda, dtype, shape):
    X = randn(*shape, dtype=dtype)
    out = run_family(kuiops.SoftmaxImpl({}), aten._softmax.default, (X, X.dim() - 1, False))
    ref = O.softmax_lastdim(to_np(X))
    assert_close_ref_bar(out, ref, dtype)
    if dtype == torch.float32:
        assert_fp32_1e5(out, ref)
    atol = 1e-3 if dtype == torch.float32 else 3e-2
    np.testing.assert_allclose(to_np(out).astype(np.float64).sum(-1), 1.0, atol=atol)


def test_softmax_unsupported(cuda):
    impl = kuiops.SoftmaxImpl({})
    X = randn(16, 16)
    assert impl.supported(aten._softmax.default, (X, 0, False), {}) is None
    assert impl.supported(aten._softmax.default, (X, 1, True), {}) is None


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("shape", [(4, 16), (2, 3, 4096), (3, 33), (2, 70000)])
def test_mean(cuda, dtype, shape):
    X = randn(*shape, dtype=dtype) + 0.25
    out = run_family(kuiops.MeanImpl({}), aten.mean.dim, (X, [-1], True))
    ref = O.mean_lastdim(to_np(X))
    assert tuple(out.shape) == shape[:-1] + (1,)
    if dtype == torch.float32:
        assert_fp32_1e5(out, ref)
    else:
        assert_close_ref_bar(out, ref, dtype)


def test_folds_all_any_max(cuda, gates):
    gates("wide")
    impl = kuiops.ReduceImpl({})
    g = torch.Generator().manual_seed(0)
    for n in (1, 31, 4096, 1_000_003):
        ones = torch.ones(n, dtype=torch.bool)
        assert bool(run_family(impl, aten.all.default, (ones.cuda(),)).item()) is True
        assert bool(run_family(impl, aten.any.default, ((~ones).cuda(),)).item()) is False
        holed = ones.clone()
        holed[n // 2] = False
        assert bool(run_family(impl, aten.all.default, (holed.cuda(),)).item()) is False
        assert bool(run_family(impl, aten.any.default, ((~holed).cuda(),)).item()) is True
        iv = torch.randint(-10 ** 12, 10 ** 12, (n,), generator=g)
        got = run_family(impl, aten.max.default, (iv.cuda(),))
        assert got.dtype == torch.int64 and int(got.item()) == int(O.reduce_fold("max", iv.numpy()))
        fv = torch.randn(n, generator=g)
        assert float(run_family(impl, aten.max.default, (fv.cuda(),)).item()) == float(fv.max())


@pytest.mark.parametrize("shape,k", [((5, 64), 10), ((3, 500), 50), ((2, 70000), 50), ((4, 9), 9), ((2, 3, 300), 7)])
def test_topk_bit_exact(cuda, gates, shape, k):
    gates("wide")
    g = torch.Generator().manual_seed(0)
    X = torch.randn(*shape, generator=g)
    vals, idx = run_family(kuiops.TopkImpl({}), aten.topk.default, (X.cuda(), k))
    rv, ri = O.topk(X.numpy(), k)
    assert_bit_exact(vals, rv)
    assert_bit_exact(idx, ri)


@pytest.mark.parametrize("case", ["few_values", "constant", "nan_inf", "negatives"])
def test_topk_ties_take_the_lowest_index(cuda, gates, case):
    gates("wide")
    g = torch.Generator().manual_seed(1)
    if case == "few_values":
        X = torch.randint(0, 8, (4, 5000), generator=g).float()
    elif case == "constant":
        X = torch.zeros(2, 9000)
    elif case == "nan_inf":
        X = torch.randn(3, 3000, generator=g)
        X[0, 5], X[0, 77], X[1, 100], X[2, 0] = float("nan"), float("inf"), float("-inf"), float("nan")
        X[2, 2999] = float("nan")
    else:
        X = -torch.rand(3, 4097, generator=g)
    vals, idx = run_family(kuiops.TopkImpl({}), aten.topk.default, (X.cuda(), 40))
    rv, ri = O.topk(X.numpy(), 40)
    assert_bit_exact(idx, ri)
    assert np.array_equal(to_np(vals), rv, equal_nan=True)


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("shape", [(5, 100), (3, 70000), (32, 128256), (300, 4099)])
def test_argmax_lowest_index_of_the_maximum(cuda, dtype, shape):
    """Row arg-max over 1..8 CTAs per row: ties (the quantised dtypes repeat values), NaN first, -0 == +0."""
    from kuipy import _ffi
    g = torch.Generator().manual_seed(3)
    X = torch.randn(*shape, generator=g).to(dtype)
    X[0, 7], X[0, shape[1] - 1] = 9.0, 9.0             # a tie between both ends of the row
    X[1, :] = 0.0
    X[1, 3] = -0.0                                      # all equal, one negative zero: index 0 wins
    X[2, shape[1] // 2] = float("nan")                  # NaN is the maximum
    X[2, shape[1] // 2 + 9] = float("nan")
    got = _ffi.argmax_lastdim(X.cuda())
    ref = torch.argmax(X.float(), dim=-1)
    assert got.dtype == torch.int64
    assert torch.equal(got.cpu(), ref)


@pytest.mark.parametrize("shape", [(1, 1), (3, 7), (5, 4097), (7, 1001), (64, 128256), (32, 2048), (4096, 33), (2, 70001)])
def test_cumsum_over_the_last_axis(cuda, gates, shape):
    """Prefix sums over one CTA or a cluster per row; rows that do not start on 16 bytes; tails."""
    gates("wide")
    impl = kuiops.DataMoveImpl({})
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(-5, 9, shape, generator=g, dtype=torch.int64)
    ids[0, 0] = (1 << 62)                                # wraps like the eager sum
    if shape[1] > 2:
        ids[0, 1] = (1 << 62)
        ids[0, 2] = (1 << 62)
    got = run_family(impl, aten.cumsum.default, (ids.cuda(), -1))
    assert got.dtype == torch.int64
    assert_bit_exact(got, O.cumsum_lastdim(ids.numpy()))
    P = torch.softmax(torch.randn(*shape, generator=g) * 3, dim=-1)      # the nucleus-sampling input
    got = run_family(impl, aten.cumsum.default, (P.cuda(), len(shape) - 1))
    assert_fp32_1e5(got, O.cumsum_lastdim(P.numpy()))
    mask = (torch.rand(*shape, generator=g) > 0.2).long()
    got = run_family(impl, aten.cumsum.default, (mask.cuda(), -1), {"dtype": torch.int64})
    assert torch.equal(got.cpu(), mask.cumsum(-1))


@pytest.mark.parametrize("shape", [(1, 1), (3, 7), (5, 4097), (300, 8193), (2, 70001), (3, 300001), (64, 128256)])
@pytest.mark.parametrize("descending", [False, True])
def test_sort_over_the_last_axis_is_the_stable_sort(cuda, gates, shape, descending):
    """Radix sort of fp32 rows: many exact ties (bf16-quantised values), NaN largest, -0 == +0, infinities;
    one tile, several tiles and ragged tails; values and permutation against the stable CPU sort."""
    gates("wide")
    impl = kuiops.DataMoveImpl({})
    g = torch.Generator().manual_seed(17)
    X = (torch.randn(*shape, generator=g) * 3).bfloat16().float()
    n = shape[1]
    if n >= 7:
        X[0, 1], X[0, n - 1] = float("nan"), float("nan")
        X[0, 2], X[0, n - 2] = float("inf"), float("-inf")
        X[-1, :] = 0.0
        X[-1, 3] = -0.0
        X[-1, n // 2] = -0.0
    if descending:
        vals, idx = run_family(impl, aten.sort.default, (X.cuda(), -1, True))
    else:
        vals, idx = run_family(impl, aten.sort.stable, (X.cuda(),), {"stable": True, "dim": len(shape) - 1})
    rv, ri = O.sort_lastdim(X.numpy(), descending)
    assert_bit_exact(idx, ri)
    assert np.array_equal(to_np(vals).view(np.uint32), rv.view(np.uint32))     # the very bits: signed zeros, NaNs
    if n == 128256:                                                            # the nucleus-sampling input
        P = torch.softmax(torch.randn(4, n, generator=g) * 3, dim=-1)
        vals, idx = run_family(impl, aten.sort.default, (P.cuda(),))
        tv, ti = torch.sort(P, dim=-1, stable=True)
        assert torch.equal(idx.cpu(), ti) and torch.equal(vals.cpu(), tv)


def test_softmax_long_rows_in_clusters(cuda):
    """64 rows of 128256 fp32: eight CTAs per row, streamed twice; and a row of -inf except one entry."""
    X = randn(64, 128256) * 3
    X[5, :] = float("-inf")
    X[5, 77] = 1.0
    out = run_family(kuiops.SoftmaxImpl({}), aten._softmax.default, (X, 1, False))
    ref = O.softmax_lastdim(to_np(X))
    assert_fp32_1e5(out, ref)
    assert float(out[5, 77]) == 1.0 and float(out[5].sum()) == 1.0


def test_topk_small_k_of_a_long_row_with_duplicates(cuda, gates):
    """k = 50 of 128256 through the thread-maxima bound; bf16-quantised values give many exact ties."""
    gates("wide")
    g = torch.Generator().manual_seed(5)
    X = (torch.randn(8, 128256, generator=g) * 3).bfloat16().float()
    X[3, 1000:1100] = X[3].max() + 1                    # 100 copies of the maximum: lowest 50 indices
    vals, idx = run_family(kuiops.TopkImpl({}), aten.topk.default, (X.cuda(), 50))
    rv, ri = O.topk(X.numpy(), 50)
    assert_bit_exact(idx, ri)
    assert_bit_exact(vals, rv)


# ---- per-token data movement (wide gates) -----------------------------------------------------------
def test_datamove_family_matches_eager(cuda, gates):
    gates("wide")
    impl = kuiops.DataMoveImpl({})
    for src in FLOATS:
        X = randn(3, 5, 1027, dtype=src)
        for dst in FLOATS:
            out = run_family(impl, aten._to_copy.default, (X,), {"dtype": dst})
            assert out.dtype == dst and torch.equal(out.cpu(), X.cpu().to(dst))
        c = run_family(impl, aten.clone.default, (X,))
        assert c.data_ptr() != X.data_ptr() and torch.equal(c, X)
        M = (randn(3, 5, 1027, seed=3) > 0.3)
        out = run_family(impl, aten.masked_fill.Scalar, (X, M, -1e4))
        assert torch.equal(out.cpu(), X.cpu().masked_fill(M.cpu(), -1e4))
        am = run_family(impl, aten.argmax.default, (X, -1))
        assert torch.equal(am.cpu(), X.cpu().float().argmax(-1))
    W = randn(50, 24, dtype=torch.bfloat16)
    ids = torch.randint(0, 50, (4, 7), generator=torch.Generator().manual_seed(2)).cuda()
    e = run_family(impl, aten.embedding.default, (W, ids))
    assert tuple(e.shape) == (4, 7, 24) and torch.equal(e.cpu(), torch.nn.functional.embedding(ids.cpu(), W.cpu()))
    # what it leaves to PyTorch
    assert impl.supported(aten._to_copy.default, (X,), {"dtype": torch.int32}) is None
    assert impl.supported(aten._to_copy.default, (X,), {"device": torch.device("cpu")}) is None
    assert impl.supported(aten._to_copy.default, (X.transpose(0, 1),), {"dtype": torch.float32}) is None
    assert impl.supported(aten.masked_fill.Scalar, (X, M[0], 0.0), {}) is None          # broadcast mask
    assert impl.supported(aten.argmax.default, (X,), {}) is None                        # flattened arg-max
    assert impl.supported(aten.argmax.default, (X, 0), {}) is None
    assert impl.supported(aten.cumsum.default, (X, -1), {}) is None                     # bf16 sums stay with PyTorch
    assert impl.supported(aten.sort.default, (X,), {}) is None                          # fp32 rows only
    gates("reference")
    from kuipy import registry
    assert aten._to_copy.default not in registry.table()


# ---- attention --------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", FLOATS)
def test_sdpa_biased(cuda, gates, dtype):
    gates("wide")
    N, H, L, S, E, Ev = 2, 3, 8, 10, 16, 12
    Q, K, V = randn(N, H, L, E, dtype=dtype), randn(N, H, S, E, dtype=dtype, seed=1), randn(N, H, S, Ev, dtype=dtype, seed=2)
    bias = randn(N, H, L, S, dtype=dtype, seed=3)
    func = aten._scaled_dot_product_efficient_attention.default
    out, lse, seed, off = run_family(kuiops.SdpaImpl({}), func, (Q, K, V, bias, True), {"scale": 0.3})
    ro, rl = O.sdpa(to_np(Q), to_np(K), to_np(V), bias=to_np(bias), scale=0.3)
    assert tuple(out.shape) == (N, H, L, Ev) and tuple(lse.shape) == (N, H, L) and lse.dtype == torch.float32
    assert_close_ref_bar(out, ro, dtype)
    assert_close_ref_bar(lse, rl, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 4, 2, 6, 9, 16), (1, 8, 2, 1, 77, 128), (2, 4, 4, 33, 33, 64), (1, 2, 1, 5, 300, 128)])
def test_sdpa_causal_grouped_query(cuda, gates, dtype, shape):
    gates("wide")
    N, H, Hkv, L, S, E = shape
    Q, K, V = randn(N, H, L, E, dtype=dtype), randn(N, Hkv, S, E, dtype=dtype, seed=1), randn(N, Hkv, S, E, dtype=dtype, seed=2)
    func = aten._scaled_dot_product_flash_attention.default
    res = run_family(kuiops.SdpaImpl({}), func, (Q, K, V, 0.0, True))
    assert len(res) == 9
    ro, rl = O.sdpa(to_np(Q), to_np(K), to_np(V), is_causal=True)
    assert_close_ref_bar(res[0], ro, dtype)
    assert_close_ref_bar(res[1], rl, dtype)
    if dtype == torch.bfloat16:
        assert_max_rel(res[0], ro, 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sdpa_efficient_overload_causal_matches_eager_under_dispatch(cuda, gates, dtype):
    """The efficient-attention overload with a causal flag, dispatched under the mode, against
    PyTorch eager: equal counts are offloaded and agree; unequal counts (ATen masks top-left there,
    the kernels bottom-right) must fall through, so the result is eager's own."""
    import kuipy
    gates("wide")
    func = aten._scaled_dot_product_efficient_attention.default
    for (L, S) in ((33, 33), (5, 33), (1, 40)):
        Q, K, V = randn(2, 4, L, 64, dtype=dtype), randn(2, 4, S, 64, dtype=dtype, seed=1), randn(2, 4, S, 64, dtype=dtype, seed=2)
        ref = func(Q, K, V, None, True, 0.0, True)
        kuipy.reset_verify()
        with kuipy.KuiperMode(verify=True):
            got = func(Q, K, V, None, True, 0.0, True)
        offloaded = str(func) in kuipy.verify_stats
        assert offloaded == (L == S)
        if offloaded:
            assert_close_ref_bar(got[0], to_np(ref[0]).astype(np.float64), dtype)
        else:
            assert torch.equal(got[0], ref[0])


def test_functional_sdpa_is_offloaded_whichever_backend_aten_picks(cuda, gates):
    """``F.scaled_dot_product_attention`` on bf16 reaches the dispatcher as the flash, the efficient or
    (on this GPU generation) the cuDNN overload; whichever it is, the call must be served by the
    kernels and agree with eager, for a causal prefill block and for a one-token decode step."""
    import kuipy
    import torch.nn.functional as F
    gates("wide")
    for (L, S, causal) in ((192, 192, True), (1, 300, False)):
        Q, K, V = randn(2, 8, L, 128, dtype=torch.bfloat16), randn(2, 2, S, 128, dtype=torch.bfloat16, seed=1), randn(2, 2, S, 128, dtype=torch.bfloat16, seed=2)
        ref = F.scaled_dot_product_attention(Q, K, V, is_causal=causal, enable_gqa=True)
        kuipy.reset_verify()
        with kuipy.KuiperMode(verify=True):
            got = F.scaled_dot_product_attention(Q, K, V, is_causal=causal, enable_gqa=True)
        served = [k for k in kuipy.verify_stats if "scaled_dot_product" in k]
        assert served, f"attention was not offloaded: {list(kuipy.verify_stats)}"
        assert sum(e["fail"] for e in kuipy.verify_stats.values()) == 0
        ro, _ = O.sdpa(to_np(Q), to_np(K), to_np(V), is_causal=causal)
        assert_max_rel(got, ro, 2e-2)
        assert got.shape == ref.shape


def test_sdpa_reference_gates_reject_causal_dropout_and_missing_bias(cuda, gates):
    gates("reference")
    impl = kuiops.SdpaImpl({})
    Q, K, V, bias = randn(1, 1, 4, 8), randn(1, 1, 4, 8), randn(1, 1, 4, 8), randn(1, 1, 4, 4)
    func = aten._scaled_dot_product_efficient_attention.default
    assert impl.supported(func, (Q, K, V, bias, True, 0.0, True), {}) is None
    assert impl.supported(func, (Q, K, V, bias, True, 0.1, False), {}) is None
    assert impl.supported(func, (Q, K, V, None, True), {}) is None
    assert impl.supported(func, (Q, K, V, bias, True), {}) is not None


# ---- data movement: bit exact ---------------------------------------------------------------------
PAYLOADS = [torch.float32, torch.bfloat16, torch.int64, torch.bool]


def payload(shape, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    if dtype == torch.bool:
        return (torch.rand(*shape, generator=g) > 0.5).cuda()
    if dtype == torch.int64:
        return torch.randint(-10 ** 15, 10 ** 15, shape, generator=g).cuda()
    return torch.randn(*shape, generator=g).to(dtype).cuda()


@pytest.mark.parametrize("dtype", PAYLOADS)
@pytest.mark.parametrize("shape,dim", [((8, 5), 1), ((8, 5), 0), ((4, 3, 6), 2), ((4, 3, 6), 1), ((2, 3, 4, 5), 0)])
def test_gather(cuda, dtype, shape, dim):
    Inp = payload(shape, dtype)
    ishape = list(shape)
    ishape[dim] = max(1, shape[dim] - 1)
    Idx = torch.randint(0, shape[dim], ishape, generator=torch.Generator().manual_seed(1)).cuda()
    out = run_family(kuiops.GatherImpl({}), aten.gather.default, (Inp, dim, Idx))
    as_np = (lambda t: t.view(torch.int16).cpu().numpy()) if dtype == torch.bfloat16 else to_np
    got = out.view(torch.int16) if dtype == torch.bfloat16 else out
    assert_bit_exact(got, O.gather(as_np(Inp), dim, to_np(Idx)))


def test_gather_smaller_index_block_and_unsupported(cuda, gates):
    gates("reference")
    impl = kuiops.GatherImpl({})
    Inp = randn(4, 4)
    assert impl.supported(aten.gather.default, (Inp, 1, torch.zeros(4, 4, device="cuda", dtype=torch.int32)), {}) is None
    assert impl.supported(aten.gather.default, (Inp, 1, torch.zeros(4, device="cuda", dtype=torch.int64)), {}) is None
    assert impl.supported(aten.gather.default, (Inp, 1, torch.zeros(4, 5, device="cuda", dtype=torch.int64)), {}) is None
    Idx = torch.randint(0, 4, (2, 3), generator=torch.Generator().manual_seed(0)).cuda()    # smaller on both axes
    assert_bit_exact(run_family(impl, aten.gather.default, (Inp, 1, Idx)), O.gather(to_np(Inp), 1, to_np(Idx)))


def _perm_index(shape, dim, seed=0):
    g = torch.Generator().manual_seed(seed)
    n = shape[dim]
    rows = int(np.prod(shape)) // n
    perm = torch.stack([torch.randperm(n, generator=g) for _ in range(rows)])
    idx = perm.reshape([s for d, s in enumerate(shape) if d != dim] + [n])
    return idx.movedim(-1, dim).contiguous()


@pytest.mark.parametrize("dtype", PAYLOADS)
@pytest.mark.parametrize("shape,dim", [((8, 5), 1), ((8, 5), 0), ((4, 3, 6), 2), ((3, 7, 2), 1)])
def test_scatter(cuda, dtype, shape, dim):
    Self, Src = payload(shape, dtype), payload(shape, dtype, seed=5)
    Idx = _perm_index(shape, dim).cuda()                  # a permutation per line: injective, as the kernel assumes
    out = run_family(kuiops.ScatterImpl({}), aten.scatter.src, (Self, dim, Idx, Src))
    as_np = (lambda t: t.view(torch.int16).cpu().numpy()) if dtype == torch.bfloat16 else to_np
    got = out.view(torch.int16) if dtype == torch.bfloat16 else out
    assert_bit_exact(got, O.scatter(as_np(Self), dim, to_np(Idx), as_np(Src)))
    assert out.data_ptr() != Self.data_ptr()


@pytest.mark.parametrize("dtype", [torch.int64, torch.bfloat16, torch.bool])
def test_gather_scatter_innermost_axis_rows_staged_on_chip(cuda, gates, dtype):
    """Rows long enough for several vector chunks, odd lengths (rows start misaligned), an index block
    smaller than the tensor on both axes, and a 3-d tensor whose outer axes merge."""
    gates("wide")
    g = torch.Generator().manual_seed(7)
    as_np = (lambda t: t.view(torch.int16).cpu().numpy()) if dtype == torch.bfloat16 else to_np
    view = (lambda t: t.view(torch.int16)) if dtype == torch.bfloat16 else (lambda t: t)
    for shape, ishape in (((70, 5001), (70, 5001)), ((70, 5001), (33, 4000)), ((3, 5, 2049), (3, 5, 2049)), ((1, 20000), (1, 20000))):
        Inp = payload(shape, dtype)
        Idx = torch.randint(0, shape[-1], ishape, generator=g).cuda()
        d = len(shape) - 1
        out = run_family(kuiops.GatherImpl({}), aten.gather.default, (Inp, d, Idx))
        assert_bit_exact(view(out), O.gather(as_np(Inp), d, to_np(Idx)))
        # scatter: a permutation prefix per row keeps the index injective
        rows = int(np.prod(ishape[:-1]))
        perm = torch.stack([torch.randperm(shape[-1], generator=g)[:ishape[-1]] for _ in range(rows)]).reshape(ishape).cuda()
        Src = payload(ishape, dtype, seed=9)
        got = run_family(kuiops.ScatterImpl({}), aten.scatter.src, (Inp, d, perm, Src))
        assert_bit_exact(view(got), O.scatter(as_np(Inp), d, to_np(perm), as_np(Src)))


def test_scatter_unsupported(cuda):
    impl = kuiops.ScatterImpl({})
    Self, Src = randn(4, 4), randn(4, 4)
    Idx = torch.zeros(4, 4, device="cuda", dtype=torch.int64)
    assert impl.supported(aten.scatter.src, (Self, 1, Idx, Src.bfloat16()), {}) is None
    assert impl.supported(aten.scatter.src, (Self, 1, Idx.int(), Src), {}) is None
    assert impl.supported(aten.scatter.src, (Self, 1, Idx, randn(4, 5)), {}) is None


@pytest.mark.parametrize("dtype", PAYLOADS)
@pytest.mark.parametrize("dim", [0, 1, 2])
def test_cat_binary(cuda, dtype, dim):
    a_shape = [4, 3, 6]
    b_shape = list(a_shape)
    b_shape[dim] += 2
    A, B = payload(a_shape, dtype), payload(b_shape, dtype, seed=1)
    out = run_family(kuiops.CatImpl({}), aten.cat.default, ([A, B], dim))
    as_np = (lambda t: t.view(torch.int16).cpu().numpy()) if dtype == torch.bfloat16 else to_np
    assert_bit_exact(out.view(torch.int16) if dtype == torch.bfloat16 else out, O.cat([as_np(A), as_np(B)], dim))


def test_cat_gates(cuda, gates):
    impl = kuiops.CatImpl({})
    A, B = randn(4, 4), randn(4, 4)
    gates("reference")
    assert impl.supported(aten.cat.default, ([A, B, A], 0), {}) is None
    assert impl.supported(aten.cat.default, ([A, randn(4, 5)], 0), {}) is None
    assert impl.supported(aten.cat.default, ([A, B.bfloat16()], 0), {}) is None
    gates("wide")
    parts = [payload((6, n), torch.int64, seed=n) for n in (3, 1, 7, 2, 5)]
    out = run_family(impl, aten.cat.default, (parts, 1))
    assert_bit_exact(out, O.cat([to_np(p) for p in parts], 1))


def test_index_and_isin(cuda, gates):
    gates("wide")
    g = torch.Generator().manual_seed(0)
    mask = (torch.rand(9, 9, generator=g) > 0.5).cuda()
    i0 = torch.randint(-9, 9, (2, 1, 5, 1), generator=g).cuda()
    i1 = torch.randint(0, 9, (1, 1, 1, 5), generator=g).cuda()
    out = run_family(kuiops.IndexImpl({}), aten.index.Tensor, (mask, [i0, i1]))
    assert_bit_exact(out, O.index(to_np(mask), 0, [to_np(i0), to_np(i1)]))
    ids = torch.randint(0, 1000, (6, 40), generator=g).cuda()
    pos = torch.randint(0, 40, (7,), generator=g).cuda()
    out = run_family(kuiops.IndexImpl({}), aten.index.Tensor, (ids, [None, pos]))
    assert_bit_exact(out, O.index(to_np(ids), 1, [to_np(pos)]))
    emb = randn(50, 3, 8, dtype=torch.bfloat16)
    rows = torch.randint(0, 50, (4, 2), generator=g).cuda()
    out = run_family(kuiops.IndexImpl({}), aten.index.Tensor, (emb, [rows]))
    assert_bit_exact(out.view(torch.int16), O.index(emb.view(torch.int16).cpu().numpy(), 0, [to_np(rows)]))
    stop = torch.randint(0, 1000, (50,), generator=g).cuda()
    assert_bit_exact(run_family(kuiops.IsinImpl({}), aten.isin.Tensor_Tensor, (ids, stop)), O.isin(to_np(ids), to_np(stop)))
    assert_bit_exact(run_family(kuiops.IsinImpl({}), aten.isin.Tensor_Tensor, (ids, stop), {"invert": True}),
                     O.isin(to_np(ids), to_np(stop), invert=True))
    big = torch.randint(0, 10 ** 6, (5000,), generator=g).cuda()          # more than one shared-memory tile
    assert_bit_exact(run_family(kuiops.IsinImpl({}), aten.isin.Tensor_Tensor, (ids * 997, big)), O.isin(to_np(ids) * 997, to_np(big)))
    scalar = torch.tensor(int(ids[0, 0]), device="cuda")
    assert_bit_exact(run_family(kuiops.IsinImpl({}), aten.isin.Tensor_Tensor, (ids, scalar)), O.isin(to_np(ids), to_np(scalar)))


def test_isin_hash_table_edges(cuda, gates):
    """INT64_MIN (the table's free-slot mark) as a test value and as an element, duplicates in the
    test set, sizes that are not multiples of the 8-element store, several passes with invert."""
    gates("wide")
    g = torch.Generator().manual_seed(4)
    lo = torch.iinfo(torch.int64).min
    ids = torch.randint(-50, 50, (3, 1001), generator=g)
    ids[0, 0], ids[2, 1000] = lo, lo
    for stop in (torch.tensor([lo, 3, 3, 7, -4]), torch.tensor([3, 7, -4]), torch.randint(-10 ** 9, 10 ** 9, (4500,), generator=g)):
        for inv in (False, True):
            got = run_family(kuiops.IsinImpl({}), aten.isin.Tensor_Tensor, (ids.cuda(), stop.cuda()), {"invert": inv})
            assert_bit_exact(got, O.isin(ids.numpy(), stop.numpy(), invert=inv))
    wide = torch.randint(-10 ** 9, 10 ** 9, (4500,), generator=g)
    pick = wide[torch.randint(0, 4500, (3, 1001), generator=g)]         # every element is in the set
    got = run_family(kuiops.IsinImpl({}), aten.isin.Tensor_Tensor, (pick.cuda(), wide.cuda()))
    assert bool(got.all())


def test_out_of_range_indices_are_skipped_and_flagged(cuda):
    from kuipy import _ffi
    Inp = randn(4, 4)
    Idx = torch.tensor([[0, 1, 2, 9]] * 4, device="cuda")
    _ffi.check_status(Inp.device)
    _ffi.gather(Inp, 1, Idx)
    assert _ffi.check_status(Inp.device) == 1
    _ffi.gather(Inp, 1, Idx.clamp(max=3))
    assert _ffi.check_status(Inp.device) == 0


# ---- elementwise ----------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("func,op", [(aten.sub.Tensor, "sub"), (aten.div.Tensor, "div"), (aten.add.Tensor, "add"), (aten.mul.Tensor, "mul")])
def test_elem_binary(cuda, dtype, func, op):
    A, B = randn(3, 5, 7, dtype=dtype), (randn(3, 5, 7, dtype=dtype, seed=1).abs() + 0.5).to(dtype)
    out = run_family(kuiops.ElementwiseImpl({}), func, (A, B))
    assert_close_ref_bar(out, O.map_op(op, to_np(A), to_np(B)), dtype)
    assert out.shape == A.shape and out.dtype == dtype


@pytest.mark.parametrize("func,c,op", [(aten.sub.Tensor, 1.5, "sub"), (aten.div.Tensor, 2.0, "div"), (aten.mul.Scalar, -3.0, "mul"),
                                       (aten.add.Scalar, 0.25, "add"), (aten.pow.Tensor_Scalar, 1.5, "pow")])
def test_elem_scalar(cuda, func, c, op):
    A = randn(4, 9).abs() + 0.1
    assert_close_ref_bar(run_family(kuiops.ElementwiseImpl({}), func, (A, c)), O.map_op(op, to_np(A), c), torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("func,op", [(aten.silu.default, "silu"), (aten.neg.default, "neg"), (aten.rsqrt.default, "rsqrt"),
                                     (aten.cos.default, "cos"), (aten.sin.default, "sin")])
def test_elem_unary(cuda, dtype, func, op):
    A = (randn(1000, dtype=dtype).abs() + 0.1).to(dtype)
    assert_close_ref_bar(run_family(kuiops.ElementwiseImpl({}), func, (A,)), O.map_op(op, to_np(A)), dtype)


def test_elem_pow2_alpha_bitwise_compare_where(cuda):
    impl = kuiops.ElementwiseImpl({})
    A, B = randn(5, 8), randn(5, 8, seed=1)
    assert_close_ref_bar(run_family(impl, aten.pow.Tensor_Scalar, (A, 2)), to_np(A).astype(np.float64) ** 2, torch.float32)
    assert_close_ref_bar(run_family(impl, aten.add.Tensor, (A, B), {"alpha": 2}), O.map_op("add", to_np(A), to_np(B), 2.0), torch.float32)
    g = torch.Generator().manual_seed(0)
    X, Y = (torch.rand(2, 6, 4, generator=g) > 0.5).cuda(), (torch.rand(2, 6, 4, generator=g) > 0.5).cuda()
    assert_bit_exact(run_family(impl, aten.bitwise_not.default, (X,)), ~to_np(X))
    assert_bit_exact(run_family(impl, aten.bitwise_and.Tensor, (X, Y)), to_np(X) & to_np(Y))
    assert_bit_exact(run_family(impl, aten.bitwise_or.Tensor, (X, Y)), to_np(X) | to_np(Y))
    for func, c, op in ((aten.le.Scalar, 0.0, "le"), (aten.lt.Scalar, 0.5, "lt"), (aten.eq.Scalar, 0.0, "eq")):
        out = run_family(impl, func, (A, c))
        assert out.dtype == torch.bool
        assert_bit_exact(out, O.compare_scalar(op, to_np(A), c))
    for dt in (torch.float32, torch.bfloat16, torch.int64):
        P, Q = payload((3, 4, 5), dt), payload((3, 4, 5), dt, seed=2)
        Cn = (torch.rand(3, 4, 5, generator=g) > 0.5).cuda()
        out = run_family(impl, aten.where.self, (Cn, P, Q))
        assert torch.equal(out.cpu(), torch.where(Cn.cpu(), P.cpu(), Q.cpu()))


def test_elem_unsupported(cuda):
    impl = kuiops.ElementwiseImpl({})
    A, B = randn(4, 4), randn(4, 4)
    assert impl.supported(aten.le.Tensor, (A, B), {}) is None
    assert impl.supported(aten.lt.Tensor, (A, B), {}) is None
    Ai = torch.ones(4, 4, device="cuda", dtype=torch.int64)
    assert impl.supported(aten.bitwise_and.Tensor, (Ai, Ai), {}) is None
    Cn = torch.ones(4, 4, device="cuda", dtype=torch.bool)
    assert impl.supported(aten.where.self, (Cn, A, randn(4, 3)), {}) is None
    assert impl.supported(aten.where.self, (Cn, A, B.bfloat16()), {}) is None
    assert impl.supported(aten.add.Tensor, (A, randn(4)), {}) is None           # no broadcasting
