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


def _tiny_hf_llama(layers=2):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=layers, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=128, vocab_size=1000, rms_norm_eps=1e-5, rope_theta=5e5,
                      max_position_embeddings=512, tie_word_embeddings=False, initializer_range=0.05)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).eval()


@pytest.mark.gpu
def test_hf_llama_through_the_backend_matches_eager(cuda, gates, monkeypatch):
    """A HuggingFace Llama (2 layers, grouped-query heads of 128) compiled with the kuiops backend:
    every layer's attention and its seven projections become kuiops nodes, the kernels really run,
    and the logits stay within the bf16 bar of the same weights evaluated in fp32 by eager."""
    import collections
    import copy
    from kuipy import _ffi
    gates("wide")
    layers = 2
    model32 = _tiny_hf_llama(layers).cuda()
    model = copy.deepcopy(model32).to(torch.bfloat16)
    ids = torch.randint(0, 1000, (2, 96), generator=torch.Generator().manual_seed(1)).cuda()
    seen = collections.Counter()
    real = inductor.lower_graph

    def spy(graph):
        n = real(graph)
        seen.update(str(node.target) for node in graph.nodes if node.op == "call_function")
        return n
    monkeypatch.setattr(inductor, "lower_graph", spy)
    with torch.no_grad():
        want = model32(ids).logits
        eager = model(ids).logits                       # the same bf16 weights through PyTorch's own kernels
        n0 = _ffi.launch_count()
        got = torch.compile(model, backend=inductor.backend)(ids).logits
    assert _ffi.launch_count() - n0 >= layers * 8
    assert seen["kuiops.sdpa.default"] >= layers, seen
    assert seen["kuiops.mm.default"] + seen["kuiops.addmm.default"] >= 4 * layers, seen
    assert inductor.call_stats["sdpa"][0] >= layers and inductor.call_stats["mm"][0] >= 4 * layers
    rel = lambda a, b: ((a.float() - b.float()).abs().max() / b.float().abs().max()).item()
    # within the bf16 bar of eager on the same weights; against the fp32 model no worse than eager bf16 itself
    # (a whole model's rounding adds up over its layers: eager bf16 is about 2.5e-2 away from fp32 here)
    assert rel(got, eager) <= 2e-2, f"max relative error {rel(got, eager):.3e} against eager bf16"
    assert rel(got, want) <= max(2e-2, 1.25 * rel(eager, want)), (rel(got, want), rel(eager, want))
    assert _ffi.tc_error() == 0


@pytest.mark.gpu
def test_hf_generate_with_compiled_forward_keeps_offloading_as_the_cache_grows(cuda, gates):
    """Greedy generation with the compiled forward: the key length changes every step, so the graph
    is compiled with symbolic sizes; the lowering must not pin it to one length (no recompilation
    per token) and the kernels must keep serving the calls."""
    import torch._dynamo
    from kuipy import _ffi
    gates("wide")
    model = _tiny_hf_llama(2).cuda().to(torch.bfloat16)
    ids = torch.randint(0, 1000, (2, 40), generator=torch.Generator().manual_seed(2)).cuda()
    with torch.no_grad():
        want = model.generate(ids, max_new_tokens=12, min_new_tokens=12, do_sample=False, pad_token_id=0)
    torch._dynamo.reset()
    model.forward = torch.compile(model.forward, backend=inductor.backend)
    served0 = inductor.call_stats.get("mm", [0, 0])[0]
    n0 = _ffi.launch_count()
    with torch.no_grad():
        got = model.generate(ids, max_new_tokens=12, min_new_tokens=12, do_sample=False, pad_token_id=0)
    assert got.shape == want.shape and torch.equal(got[:, :40], ids)
    # 12 forwards x 2 layers x 7 projections, were every step served by the kernels
    assert inductor.call_stats["mm"][0] - served0 >= 10 * 2 * 7
    assert _ffi.launch_count() - n0 >= 10 * 2 * 8
    assert _ffi.tc_error() == 0
