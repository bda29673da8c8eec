"""The ``supported()`` gates against the reference's recorded decisions (CPU only).

``tests/golden/supported_golden.json`` holds what the reference's own gates answered for every
call in ``tests/golden/gate_cases.py`` (recorded by ``gen_supported_golden.py``).  With
``config.GATES == "reference"`` this repository must give the same answer, except where the new
kernels have no fp64 / unsigned path; with "wide" gates every call the reference accepts must
still be accepted.
"""
import json
from pathlib import Path

import pytest
import torch

from fake_cuda import FakeCudaTensor
from gate_cases import DT, cases

from kuipy import kuiops

GOLD = json.loads((Path(__file__).parent / "golden" / "supported_golden.json").read_text())


def _mat(d):
    if isinstance(d, tuple) and d and d[0] == "T":
        return FakeCudaTensor(torch.zeros(d[1], dtype=DT[d[2]]))
    if isinstance(d, tuple) and d and d[0] == "CPU":
        return torch.zeros(d[1], dtype=DT[d[2]])
    if isinstance(d, tuple) and d and d[0] == "L":
        return [_mat(x) for x in d[1]]
    return d


def _op(name):
    packet, overload = name.split(".")
    return getattr(getattr(torch.ops.aten, packet), overload)


def _uses_f64(args):
    def walk(d):
        if isinstance(d, tuple) and d and d[0] in ("T", "CPU"):
            return d[2] == "f64"
        if isinstance(d, tuple) and d and d[0] == "L":
            return any(walk(x) for x in d[1])
        return False
    return any(walk(a) for a in args)


def _decide(fams, fam, op, args, kwargs):
    impl = fams.setdefault(fam, getattr(kuiops, fam)({}))
    return impl.supported(_op(op), tuple(_mat(a) for a in args), dict(kwargs)) is not None


def test_case_list_matches_golden():
    cs = cases()
    assert len(cs) == len(GOLD["cases"])
    for c, g in zip(cs, GOLD["cases"]):
        assert (c[0], c[1]) == (g["family"], g["op"])


def test_reference_gates_reproduce_reference_decisions(gates):
    gates("reference")
    fams, diffs = {}, []
    for (fam, op, args, kwargs), g in zip(cases(), GOLD["cases"]):
        got = _decide(fams, fam, op, args, kwargs)
        if got != g["accept"]:
            if g["accept"] and _uses_f64(args):
                continue        # documented: no fp64 kernels
            diffs.append((fam, op, args, kwargs, g["accept"], got))
    assert not diffs, f"{len(diffs)} decisions differ from the reference, first: {diffs[0]}"


def test_wide_gates_accept_everything_the_reference_accepts(gates):
    gates("wide")
    fams, lost = {}, []
    for (fam, op, args, kwargs), g in zip(cases(), GOLD["cases"]):
        if g["accept"] and not _uses_f64(args) and not _decide(fams, fam, op, args, kwargs):
            lost.append((fam, op, args))
    assert not lost, f"wide gates reject calls the reference takes: {lost[:3]}"


def test_wide_gates_take_the_decode_shapes(gates):
    gates("wide")
    aten = torch.ops.aten
    f = lambda s, dt=torch.bfloat16: FakeCudaTensor(torch.zeros(s, dtype=dt))
    assert kuiops.MmImpl({}).supported(aten.mm.default, (f((16, 4096)), f((4096, 4096))), {}) is not None
    assert kuiops.MmImpl({}).supported(aten.mm.default, (f((17, 9)), f((9, 13))), {}) is not None
    assert kuiops.AddmmImpl({}).supported(aten.addmm.default, (f((64,)), f((8, 32)), f((32, 64))), {}) is not None
    assert kuiops.CatImpl({}).supported(aten.cat.default, ([f((64, 512), torch.int64)] * 8, 1), {}) is not None
    q, k, v = f((2, 8, 1, 128)), f((2, 2, 77, 128)), f((2, 2, 77, 128))
    sd = kuiops.SdpaImpl({})
    assert sd.supported(aten._scaled_dot_product_flash_attention.default, (q, k, v, 0.0, True), {}) is not None
    # a decode step reaches the efficient overload without a causal flag (one query row sees every key)
    assert sd.supported(aten._scaled_dot_product_efficient_attention.default, (q, k, v, None, True, 0.0, False), {}) is not None
    assert sd.supported(aten._scaled_dot_product_flash_attention.default, (q, k, v, 0.1, True), {}) is None


@pytest.mark.parametrize("rec", GOLD["tiles"], ids=lambda r: f"{r['dtype']}-{r['M']}x{r['N']}x{r['K']}")
def test_tile_choosers_match_reference(rec):
    dt = DT[rec["dtype"]]
    assert kuiops._bt2d_tile(dt, rec["M"], rec["N"], rec["K"]) == rec["bt2d"]
    assert kuiops._tc2d_tile(dt, rec["M"], rec["N"], rec["K"]) == rec["tc2d"]


def test_new_families_gate_like_torch_signatures(gates):
    gates("wide")
    aten = torch.ops.aten
    f = lambda s, dt=torch.float32: FakeCudaTensor(torch.zeros(s, dtype=dt))
    tk = kuiops.TopkImpl({})
    assert tk.supported(aten.topk.default, (f((64, 128256)), 50), {}) is not None
    assert tk.supported(aten.topk.default, (f((64, 128256)), 50, 0), {}) is None          # not the last axis
    assert tk.supported(aten.topk.default, (f((64, 128256)), 50, -1, False), {}) is None  # smallest
    assert tk.supported(aten.topk.default, (f((4, 10)), 11), {}) is None                  # k > n
    assert tk.supported(aten.topk.default, (f((4, 10), torch.bfloat16), 3), {}) is None
    isn = kuiops.IsinImpl({})
    assert isn.supported(aten.isin.Tensor_Tensor, (f((64, 2048), torch.int64), f((1024,), torch.int64)), {}) is not None
    assert isn.supported(aten.isin.Tensor_Tensor, (f((8,), torch.int64), f((), torch.int64)), {}) is not None
    assert isn.supported(aten.isin.Tensor_Tensor, (f((8,), torch.int32), f((4,), torch.int64)), {}) is None
    ix = kuiops.IndexImpl({})
    i4 = f((2, 1, 5, 5), torch.int64)
    assert ix.supported(aten.index.Tensor, (f((9, 9), torch.bool), [i4, i4]), {}) is not None
    assert ix.supported(aten.index.Tensor, (f((64, 2048), torch.int64), [None, f((7,), torch.int64)]), {}) is not None
    assert ix.supported(aten.index.Tensor, (f((4, 4, 4)), [f((2,), torch.int64), None, f((2,), torch.int64)]), {}) is None
    assert ix.supported(aten.index.Tensor, (f((4, 4)), [f((4, 4), torch.bool)]), {}) is None   # mask indexing
    rd = kuiops.ReduceImpl({})
    assert rd.supported(aten.all.default, (f((4, 4), torch.bool),), {}) is not None
    assert rd.supported(aten.any.default, (f((9,), torch.bool),), {}) is not None
    assert rd.supported(aten.max.default, (f((9,), torch.int64),), {}) is not None
    assert rd.supported(aten.max.default, (f((9,), torch.bfloat16),), {}) is None


def test_datamove_gates_on_metadata_only():
    """What the per-token data-movement family takes and what it leaves to PyTorch (no GPU: the
    gates only read tensor metadata)."""
    aten = torch.ops.aten
    impl = kuiops.DataMoveImpl({})
    X = FakeCudaTensor(torch.zeros(4, 6, 64, dtype=torch.bfloat16))
    M = FakeCudaTensor(torch.zeros(4, 6, 64, dtype=torch.bool))
    ids = FakeCudaTensor(torch.zeros(3, 5, dtype=torch.int64))
    W = FakeCudaTensor(torch.zeros(100, 32, dtype=torch.float16))
    assert impl.supported(aten._to_copy.default, (X,), {"dtype": torch.float32})[:2] == ("cast", torch.float32)
    assert impl.supported(aten._to_copy.default, (X,), {})[:2] == ("cast", torch.bfloat16)
    assert impl.supported(aten.clone.default, (X,), {})[0] == "cast"
    assert impl.supported(aten.masked_fill.Scalar, (X, M, -3.0), {})[:2] == ("masked_fill", -3.0)
    assert impl.supported(aten.argmax.default, (X, 2), {})[0] == "argmax"
    assert impl.supported(aten.embedding.default, (W, ids), {})[0] == "embedding"
    F = FakeCudaTensor(torch.zeros(4, 6, 64, dtype=torch.float32))
    assert impl.supported(aten.cumsum.default, (ids, -1), {})[0] == "cumsum"
    assert impl.supported(aten.cumsum.default, (F, 2), {"dtype": torch.float32})[0] == "cumsum"
    assert impl.supported(aten.sort.default, (F,), {})[:2] == ("sort", False)
    assert impl.supported(aten.sort.default, (F, -1, True), {})[:2] == ("sort", True)
    assert impl.supported(aten.sort.stable, (F,), {"stable": True, "dim": 2, "descending": True})[:2] == ("sort", True)
    # left to PyTorch
    assert impl.supported(aten._to_copy.default, (X,), {"dtype": torch.int64}) is None
    assert impl.supported(aten._to_copy.default, (X,), {"dtype": torch.float32, "device": torch.device("cpu")}) is None
    assert impl.supported(aten._to_copy.default, (torch.zeros(4, 4),), {"dtype": torch.bfloat16}) is None      # not on the GPU
    assert impl.supported(aten.clone.default, (X,), {"memory_format": torch.channels_last}) is None
    assert impl.supported(aten.masked_fill.Scalar, (X, FakeCudaTensor(torch.zeros(6, 64, dtype=torch.bool)), 0.0), {}) is None
    assert impl.supported(aten.masked_fill.Scalar, (X, M, True), {}) is None
    assert impl.supported(aten.argmax.default, (X,), {}) is None and impl.supported(aten.argmax.default, (X, 1), {}) is None
    assert impl.supported(aten.argmax.default, (X, -1, True), {}) is None
    assert impl.supported(aten.cumsum.default, (ids, 0), {}) is None                                  # not the last axis
    assert impl.supported(aten.cumsum.default, (ids, -1), {"dtype": torch.float32}) is None           # converting sum
    assert impl.supported(aten.cumsum.default, (X, -1), {}) is None                                   # 16-bit floats
    assert impl.supported(aten.sort.default, (F, 0), {}) is None and impl.supported(aten.sort.default, (X,), {}) is None
    assert impl.supported(aten.sort.stable, (F,), {"stable": False, "dim": 1}) is None
    assert impl.supported(aten.embedding.default, (W, FakeCudaTensor(torch.zeros(3, dtype=torch.int32))), {}) is None



def test_efficient_attention_causal_needs_square_scores(gates):
    """ATen masks the efficient overload top-left, the kernels mask bottom-right: with a causal
    flag the two only agree for equal query and key counts, so other shapes must fall through.
    The flash overload is bottom-right in ATen too and is taken either way."""
    gates("wide")
    aten = torch.ops.aten
    impl = kuiops.SdpaImpl({})
    q = lambda l: FakeCudaTensor(torch.zeros((2, 4, l, 64), dtype=torch.bfloat16))
    eff, fl = aten._scaled_dot_product_efficient_attention.default, aten._scaled_dot_product_flash_attention.default
    assert impl.supported(eff, (q(8), q(8), q(8), None, True, 0.0, True), {}) is not None
    assert impl.supported(eff, (q(5), q(8), q(8), None, True, 0.0, True), {}) is None
    assert impl.supported(eff, (q(1), q(8), q(8), None, True, 0.0, True), {}) is None
    assert impl.supported(eff, (q(5), q(8), q(8), None, True, 0.0, False), {}) is not None
    assert impl.supported(fl, (q(5), q(8), q(8), 0.0, True), {}) is not None
