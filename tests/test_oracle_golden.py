"""Pin the CPU oracle: every restatement in ``oracle/kuiops_oracle.py`` against the golden
vectors PyTorch eager produced (``tests/golden/ops_golden.npz``) and against the reference's own
verify-mode metric (``tests/golden/verify_golden.json``).  CPU only."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import kuiops_oracle as O

G = np.load(Path(__file__).parent / "golden" / "ops_golden.npz")
F64_TOL = dict(rtol=1e-5, atol=1e-5)     # golden outputs are fp32 eager results


def test_gemm_family():
    np.testing.assert_allclose(O.mm(G["mm_A"], G["mm_B"]), G["mm_out"], **F64_TOL)
    np.testing.assert_allclose(O.addmm(G["addmm_C"], G["mm_A"], G["mm_B"], 0.5, 2.0), G["addmm_out"], **F64_TOL)
    np.testing.assert_allclose(O.addmm(G["addmm_bias"], G["mm_A"], G["mm_B"]), G["addmm_bias_out"], **F64_TOL)
    np.testing.assert_allclose(O.bmm(G["bmm_A"], G["bmm_B"]), G["bmm_out"], **F64_TOL)


def test_softmax_and_mean():
    np.testing.assert_allclose(O.softmax_lastdim(G["softmax_X"]), G["softmax_out"], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(O.mean_lastdim(G["softmax_X"]), G["mean_out"], rtol=1e-5, atol=1e-6)


def test_attention_biased_and_lse():
    out, lse = O.sdpa(G["sdpa_Q"], G["sdpa_K"], G["sdpa_V"], bias=G["sdpa_bias"], scale=0.3)
    np.testing.assert_allclose(out, G["sdpa_out"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(lse, G["sdpa_lse"], rtol=1e-5, atol=1e-5)


def test_attention_causal_grouped_query():
    out, _ = O.sdpa(G["gqa_Q"], G["gqa_K"], G["gqa_V"], is_causal=True)
    np.testing.assert_allclose(out, G["gqa_out"], rtol=1e-4, atol=1e-5)


def test_data_movement_bit_exact():
    assert np.array_equal(O.gather(G["gather_inp"], 2, G["gather_idx"]), G["gather_out"])
    assert np.array_equal(O.gather(G["gather_inp"], 0, G["gather0_idx"]), G["gather0_out"])
    assert np.array_equal(O.gather_fast(G["gather_inp"], 2, G["gather_idx"]), G["gather_out"])
    assert np.array_equal(O.gather_fast(G["gather_inp"], 0, G["gather0_idx"]), G["gather0_out"])
    assert np.array_equal(O.scatter(G["gather_inp"], 2, G["scatter_idx"], G["scatter_src"]), G["scatter_out"])
    assert np.array_equal(O.scatter_fast(G["gather_inp"], 2, G["scatter_idx"], G["scatter_src"]), G["scatter_out"])
    assert np.array_equal(O.cat([G["cat_a"], G["cat_b"]], 1), G["cat_out"])
    assert np.array_equal(O.index(G["index_self"], 0, [G["index_i0"], G["index_i1"]]), G["index_out"])
    assert np.array_equal(O.index(G["index2_self"], 1, [G["index2_pos"]]), G["index2_out"])
    assert np.array_equal(O.isin(G["index2_self"], G["isin_test"]), G["isin_out"])
    assert np.array_equal(O.isin(G["index2_self"], G["isin_test"], invert=True), ~G["isin_out"])


def test_topk_tie_order_and_values():
    v, i = O.topk(G["topk_X"], 10)
    assert np.array_equal(v, G["topk_vals"]) and np.array_equal(i, G["topk_idx"])
    v2, i2 = O.topk(G["topk2_X"], 50)
    assert np.array_equal(v2, G["topk2_vals"]) and np.array_equal(i2, G["topk2_idx"])


def test_topk_nan_ranks_first():
    x = np.array([[1.0, np.nan, np.inf, 3.0, np.nan]], dtype=np.float32)
    v, i = O.topk(x, 3)
    assert list(i[0]) == [1, 4, 2] and np.isnan(v[0, 0]) and np.isnan(v[0, 1]) and v[0, 2] == np.inf
    tv, ti = torch.topk(torch.from_numpy(x), 3)
    assert sorted(ti[0].tolist()[:2]) == [1, 4] and ti[0, 2].item() == 2


def test_maps():
    X, Y = G["map_X"], G["map_Y"]
    tol = dict(rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(O.map_op("silu", X), G["map_silu"], **tol)
    np.testing.assert_allclose(O.map_op("rsqrt", Y), G["map_rsqrt"], **tol)
    np.testing.assert_allclose(O.map_op("pow", Y, 1.5), G["map_pow"], **tol)
    np.testing.assert_allclose(O.map_op("add", X, Y, alpha=2.0), G["map_add_alpha"], **tol)
    np.testing.assert_allclose(O.map_op("div", X, Y), G["map_div"], **tol)
    np.testing.assert_allclose(O.map_op("sub", X, 1.5), G["map_sub_scalar"], **tol)
    np.testing.assert_allclose(O.map_op("gelu", X), G["map_gelu"], **tol)
    assert np.array_equal(O.compare_scalar("le", X, 0.0), G["map_le"])
    assert np.array_equal(O.where(X > 0, X, Y), G["map_where"])


def test_folds():
    assert bool(O.reduce_fold("all", G["fold_bool"])) == bool(G["fold_all"])
    assert bool(O.reduce_fold("any", G["fold_bool"])) == bool(G["fold_any"])
    assert int(O.reduce_fold("max", G["fold_i64"])) == int(G["fold_max"])


def test_rmsnorm_and_rope_against_torch():
    g = torch.Generator().manual_seed(1)
    x, w = torch.randn(5, 64, generator=g), torch.randn(64, generator=g)
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w
    y, _ = O.rmsnorm(x.numpy(), w.numpy(), 1e-5)
    np.testing.assert_allclose(y, ref.numpy(), rtol=1e-5, atol=1e-6)
    q = torch.randn(7, 2, 16, generator=g)
    pos = torch.arange(3, 10)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 16, 2).float() / 16))
    ang = pos[:, None].float() * inv[None]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, None], torch.cat([ang.sin(), ang.sin()], -1)[:, None]
    rot = torch.cat([-q[..., 8:], q[..., :8]], -1)
    np.testing.assert_allclose(O.rope(q.numpy(), pos.numpy(), 10000.0), (q * cos + rot * sin).numpy(), rtol=1e-5, atol=1e-5)


def test_comparator_matches_reference_verify_metric():
    rec = json.loads((Path(__file__).parent / "golden" / "verify_golden.json").read_text())
    g = torch.Generator().manual_seed(rec["seed"])
    for r in rec["records"]:
        a = torch.randn(*rec["shape"], generator=g)
        b = a + r["noise"] * torch.randn(*rec["shape"], generator=g)
        rel = O.rel_frobenius(a.numpy(), b.numpy())
        assert rel == pytest.approx(r["max_rel"], rel=1e-4, abs=1e-9)
        assert (rel > rec["tol"]) == bool(r["fail"])


def test_sort_and_cumsum_against_eager():
    """The sampling-tail restatements against PyTorch eager on CPU (seeded): the stable sort with its
    NaN / signed-zero / infinity rules in both directions, and the prefix sums."""
    g = torch.Generator().manual_seed(9)
    X = (torch.randn(6, 777, generator=g) * 3).bfloat16().float()        # quantised: many exact ties
    X[0, 3] = X[0, 500] = float("nan")
    X[1, :] = 0.0
    X[1, 5] = X[1, 600] = -0.0
    X[2, 7], X[2, 9] = float("inf"), float("-inf")
    for desc in (False, True):
        v, i = O.sort_lastdim(X.numpy(), desc)
        tv, ti = torch.sort(X, dim=-1, descending=desc, stable=True)
        assert np.array_equal(i, ti.numpy())
        assert np.array_equal(v.view(np.uint32), tv.numpy().view(np.uint32))
    ids = torch.randint(-9, 9, (5, 301), generator=g)
    assert np.array_equal(O.cumsum_lastdim(ids.numpy()), ids.cumsum(-1).numpy())
    P = torch.softmax(torch.randn(4, 5000, generator=g), -1)
    np.testing.assert_allclose(O.cumsum_lastdim(P.numpy()), P.double().cumsum(-1).float().numpy(), rtol=1e-6, atol=1e-7)
