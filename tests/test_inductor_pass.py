"""The graph-level front end (``kuipy.inductor``): aten nodes of an FX graph traced on fake CUDA
tensors are rewritten to ``kuiops::*`` custom ops exactly where ``supported()`` says so.  The
rewrite itself needs no GPU; the end-to-end compile test does."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode
from torch.fx.experimental.proxy_tensor import make_fx

from kuipy import inductor


def _trace(fn, *shapes_dtypes):
    mode = FakeTensorMode()
    with mode:
        args = [torch.empty(s, device="cuda", dtype=d) for s, d in shapes_dtypes]
    return make_fx(fn, tracing_mode="fake")(*args)


def _targets(gm):
    return [str(n.target) for n in gm.graph.nodes if n.op == "call_function"]


def test_sampling_graph_is_lowered(gates):
    gates("wide")

    def f(h, w, ids, stop):
        logits = torch.mm(h, w.t()).float()
        p = torch.softmax(logits, -1)
        v, i = torch.topk(p, 5)
        tok = torch.gather(i, 1, torch.zeros_like(i[:, :1]))
        return torch.cat([ids, tok], 1), torch.isin(tok, stop), v.mean(-1, keepdim=True)
    gm = _trace(f, ((8, 64), torch.bfloat16), ((1000, 64), torch.bfloat16), ((8, 3), torch.int64), ((4,), torch.int64))
    n = inductor.lower_graph(gm.graph)
    gm.recompile()
    t = _targets(gm)
    assert n >= 6
    for name in ("kuiops.mm", "kuiops.softmax", "kuiops.topk", "kuiops.gather", "kuiops.cat", "kuiops.isin", "kuiops.mean_dim"):
        assert any(name in x for x in t), (name, t)
    assert not any("aten.mm" in x or "aten._softmax" in x or "aten.topk" in x for x in t)
    # fake propagation through the custom ops still works (shapes, dtypes)
    mode = FakeTensorMode()
    with mode:
        outs = gm(torch.empty(8, 64, device="cuda", dtype=torch.bfloat16), torch.empty(1000, 64, device="cuda", dtype=torch.bfloat16),
                  torch.empty(8, 3, device="cuda", dtype=torch.int64), torch.empty(4, device="cuda", dtype=torch.int64))
    assert outs[0].shape == (8, 4) and outs[1].dtype == torch.bool and outs[2].shape == (8, 1)


def test_nucleus_sampling_tail_is_lowered(gates):
    """sort -> softmax -> cumsum -> argmax of the top-p filter; the mask arithmetic stays with the compiler."""
    gates("wide")

    def f(logits):
        s, i = torch.sort(logits, descending=False)
        c = torch.softmax(s, -1).cumsum(-1)
        keep = c > 0.1
        return torch.argmax(torch.where(keep, s, torch.full_like(s, -1e9)), -1), i
    gm = _trace(f, ((8, 1000), torch.float32))
    n = inductor.lower_graph(gm.graph)
    gm.recompile()
    t = _targets(gm)
    assert n == 4, t
    for name in ("kuiops.sort", "kuiops.softmax", "kuiops.cumsum", "kuiops.argmax"):
        assert any(name in x for x in t), (name, t)
    assert any("aten.gt" in x for x in t) and any("aten.where" in x for x in t)
    with FakeTensorMode():
        tok, perm = gm(torch.empty(8, 1000, device="cuda", dtype=torch.float32))
    assert tok.shape == (8,) and tok.dtype == torch.int64 and perm.shape == (8, 1000) and perm.dtype == torch.int64
    # bf16 rows are not sorted by the kernels: the node stays
    gm = _trace(lambda x: torch.sort(x)[0], ((8, 1000), torch.bfloat16))
    assert inductor.lower_graph(gm.graph) == 0


def test_reference_gates_leave_unsupported_nodes_alone(gates):
    gates("reference")
    gm = _trace(lambda a, b: torch.mm(a, b), ((128, 63), torch.float32), ((63, 128), torch.float32))
    assert inductor.lower_graph(gm.graph) == 0 and any("aten.mm" in x for x in _targets(gm))
    gm = _trace(lambda a, b: torch.mm(a, b), ((128, 64), torch.float32), ((64, 128), torch.float32))
    assert inductor.lower_graph(gm.graph) == 1


def test_cpu_graphs_are_never_lowered(gates):
    gates("wide")
    gm = make_fx(lambda a, b: torch.mm(a, b))(torch.randn(8, 8), torch.randn(8, 8))
    assert inductor.lower_graph(gm.graph) == 0


def test_attention_node_is_lowered(gates):
    gates("wide")

    def f(q, k, v):
        return torch.ops.aten._scaled_dot_product_flash_attention.default(q, k, v, 0.0, True)[0]
    gm = _trace(f, ((2, 8, 128, 128), torch.bfloat16), ((2, 2, 128, 128), torch.bfloat16), ((2, 2, 128, 128), torch.bfloat16))
    assert inductor.lower_graph(gm.graph) == 1
    gm.recompile()
    assert any("kuiops.sdpa" in x for x in _targets(gm)) and not any("flash_attention" in x for x in _targets(gm))


@pytest.mark.gpu
def test_compiled_function_runs_on_kuiops(cuda, gates):
    gates("wide")
    from kuipy import _ffi

    def f(h, w):
        return torch.softmax(torch.mm(h, w.t()).float(), -1)
    g = torch.Generator().manual_seed(0)
    h = torch.randn(16, 256, generator=g).bfloat16().cuda()
    w = (torch.randn(512, 256, generator=g) / 16).bfloat16().cuda()
    n0 = _ffi.launch_count()
    out = torch.compile(f, backend=inductor.backend)(h, w)
    assert _ffi.launch_count() - n0 >= 2
    ref = f(h, w)
    assert torch.allclose(out, ref, rtol=2e-2, atol=1e-4)
