"""The GEMM plan tuner behind ``KUIPY_RE_TUNE`` (kuipy.tuner): table persistence and the
library-side plan table on CPU; timing of real plans and the lazy first-call path on a GPU."""
import json

import pytest
import torch

from kuipy import _ffi, tuner
import kuipy.config as C


@pytest.fixture
def clean_table():
    saved = dict(tuner._plans)
    yield
    _ffi.lib().kuiops_gemm_tune_clear()
    tuner._plans.clear()
    tuner.apply(saved, _ffi.lib())


def test_candidates_respect_the_kernel_limits():
    assert tuner.candidates(32, 4096, 4096, 0) == [(1, 0), (2, 0), (3, 0), (4, 0), (8, 0)]
    assert tuner.candidates(32, 6144, 4096, 2)[0] == (2, 0)             # rotary epilogue needs a split
    assert tuner.candidates(16, 512, 128, 0) == [(1, 0), (2, 0)]         # two k-blocks: at most two slices
    assert tuner.candidates(4096, 4096, 4096, 0) == [(0, 128), (0, 256)]
    assert tuner.candidates(4096, 128, 4096, 0) == [(0, 128)]


def test_library_table_overrides_and_forgets_a_plan(clean_table):
    L = _ffi.lib()
    rule = _ffi.gemm_plan(torch.bfloat16, 32, 4096, 4096)
    assert rule[2] is True and 1 <= rule[0] <= 8
    rule_swiglu = _ffi.gemm_plan(torch.bfloat16, 32, 4096, 4096, epilogue=1)
    other = 4 if rule[0] != 4 else 2
    assert L.kuiops_gemm_tune_set(_ffi.BF16, 0, 1, 32, 4096, 4096, other, 0) == 0
    assert _ffi.gemm_plan(torch.bfloat16, 32, 4096, 4096)[0] == other
    assert _ffi.gemm_plan(torch.bfloat16, 32, 4096, 4096, epilogue=1) == rule_swiglu      # keyed by epilogue too
    assert _ffi.gemm_plan(torch.bfloat16, 16, 4096, 4096)[1] == 16           # other shapes keep the rule
    assert L.kuiops_gemm_tune_set(_ffi.BF16, 0, 1, 32, 4096, 4096, 0, 0) == 0
    assert _ffi.gemm_plan(torch.bfloat16, 32, 4096, 4096) == rule
    # normal placement: the column tile
    assert L.kuiops_gemm_tune_set(_ffi.BF16, 0, 1, 4096, 4096, 4096, 0, 128) == 0
    assert _ffi.gemm_plan(torch.bfloat16, 4096, 4096, 4096)[1:] == (128, False)
    # refused: fp32 has no tensor-core plan, nine slices exceed a cluster, 64 is not a tile
    assert L.kuiops_gemm_tune_set(_ffi.F32, 0, 1, 32, 4096, 4096, 2, 0) == _ffi.EUNSUPPORTED
    assert L.kuiops_gemm_tune_set(_ffi.BF16, 0, 1, 32, 4096, 4096, 9, 0) == _ffi.EINVAL
    assert L.kuiops_gemm_tune_set(_ffi.BF16, 0, 1, 4096, 4096, 4096, 0, 64) == _ffi.EINVAL
    # a split beyond the number of k-blocks is ignored, not applied
    assert L.kuiops_gemm_tune_set(_ffi.BF16, 0, 1, 8, 512, 64, 4, 0) == 0
    assert _ffi.gemm_plan(torch.bfloat16, 8, 512, 64)[0] == 1


def test_tables_round_trip_and_user_entries_override_shipped_ones(tmp_path, monkeypatch, clean_table):
    shipped, user = tmp_path / "shipped.json", tmp_path / "cache" / "tune_params.json"
    k1, k2 = tuner.key_of(_ffi.BF16, 0, True, 32, 4096, 4096), tuner.key_of(_ffi.BF16, 1, True, 32, 28672, 4096)
    shipped.write_text(json.dumps({"MM": {"impl": "tc2d", "plans": {k1: {"splits": 4, "bn": 0}, k2: {"splits": 2, "bn": 0}}}}))
    monkeypatch.setattr(tuner, "SHIPPED", shipped)
    monkeypatch.setattr(C, "TUNE_FILE", user)
    assert tuner.load_tables() == {k1: {"splits": 4, "bn": 0}, k2: {"splits": 2, "bn": 0}}
    user.parent.mkdir()
    user.write_text(json.dumps({"MM": {"plans": {k1: {"splits": 8, "bn": 0}}}, "SOFTMAX": [1, 2]}))
    plans = tuner.load_tables()
    assert plans[k1]["splits"] == 8 and plans[k2]["splits"] == 2
    _ffi.lib().kuiops_gemm_tune_clear()
    tuner._plans.clear()
    assert tuner.apply(plans, _ffi.lib()) == 2
    assert _ffi.gemm_plan(torch.bfloat16, 32, 4096, 4096)[0] == 8
    assert _ffi.gemm_plan(torch.bfloat16, 32, 28672, 4096, epilogue=1)[0] == 2
    tuner.save()
    back = json.loads(user.read_text())
    assert back["SOFTMAX"] == [1, 2] and back["MM"]["plans"][k2]["splits"] == 2      # other families' entries survive
    # a damaged file is an empty table, not an error
    user.write_text("{ not json")
    assert tuner.load_tables()[k1]["splits"] == 4


def test_family_hook_passes_the_table_through_without_a_gpu():
    from kuipy import kuiops
    if torch.cuda.is_available():
        pytest.skip("the CPU behaviour of the hook")
    key = tuner.key_of(_ffi.BF16, 0, True, 32, 4096, 4096)
    fam = kuiops.MmImpl({"MM": {"impl": "tc2d", "plans": {key: {"splits": 4, "bn": 0}}}})
    out = fam.tune({})
    assert out["MM"]["plans"][key]["splits"] == 4 and out["MM"]["impl"] == "tc2d"


@pytest.mark.gpu
def test_tuner_times_plans_and_the_result_stays_correct(cuda, clean_table):
    from oracle import kuiops_oracle as O
    from _util import to_np
    plan = tuner.tune_gemm(torch.bfloat16, 32, 4096, 4096, True, 0, iters=10)
    assert set(plan["tried"]) >= {"rule", "splits=1", "splits=8"} and plan["us"] <= plan["tried"]["rule"] * 1.001
    assert all(v > 0 for v in plan["tried"].values())
    g = torch.Generator().manual_seed(0)
    A = torch.randn(32, 4096, generator=g).bfloat16().cuda()
    W = (torch.randn(4096, 4096, generator=g) / 64).bfloat16().cuda()
    ref = O.mm(to_np(A), to_np(W).T)
    for splits in (1, 2, 3, 4, 8, 0):                                   # every plan the tuner may install gives the same product
        assert _ffi.lib().kuiops_gemm_tune_set(_ffi.BF16, 0, 1, 32, 4096, 4096, splits, 0) == 0
        assert O.max_rel_err(to_np(_ffi.gemm(A, W, trans_b=True)), ref) <= 2e-2
    A2 = torch.randn(4096, 512, generator=g).bfloat16().cuda()
    W2 = (torch.randn(1024, 512, generator=g) / 23).bfloat16().cuda()
    outs = []
    for bn in (128, 256):
        assert _ffi.lib().kuiops_gemm_tune_set(_ffi.BF16, 0, 1, 4096, 1024, 512, 0, bn) == 0
        outs.append(_ffi.gemm(A2, W2, trans_b=True))
    assert torch.equal(outs[0], outs[1])                                # the column tile does not change a bit
    assert _ffi.tc_error() == 0


@pytest.mark.gpu
def test_re_tune_flag_tunes_a_new_shape_at_first_use_and_saves(cuda, tmp_path, monkeypatch, clean_table):
    monkeypatch.setattr(C, "TUNE_FILE", tmp_path / "tune_params.json")
    monkeypatch.setattr(C, "RE_TUNE", True)
    A = torch.randn(8, 1024, device="cuda").bfloat16()
    W = torch.randn(2048, 1024, device="cuda").bfloat16()
    key = tuner.key_of(_ffi.BF16, 0, True, 8, 2048, 1024)
    tuner._plans.pop(key, None)
    out = _ffi.gemm(A, W, trans_b=True)
    saved = json.loads((tmp_path / "tune_params.json").read_text())
    assert key in saved["MM"]["plans"] and "tried" in saved["MM"]["plans"][key]
    assert torch.equal(out, _ffi.gemm(A, W, trans_b=True))              # second call: no tuning, same plan, same bits
