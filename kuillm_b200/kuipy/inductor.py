"""Graph-level front end: lower aten nodes of an FX graph to kuiops custom ops.

The reference only intercepts eagerly (``TorchDispatchMode``, kuipy/__init__.py:133-178 there); it
has no compiler pass.  This module is a second front end over the same op table: every aten
overload in the table gets a ``torch.library`` custom op ``kuiops::<name>`` (CUDA implementation =
``registry.try_dispatch``; fake implementation = the aten op on fake tensors, so shapes and dtypes
propagate), and ``lower_graph`` rewrites an aten-level ``torch.fx.Graph`` in place, consulting the
same ``supported()`` gates on the nodes' fake-tensor metadata.  Two ways to use it:

* ``install_inductor_pass()`` registers ``lower_graph`` as Inductor's post-grad custom pass, so
  ``torch.compile(model)`` keeps Inductor's fusion for elementwise code and calls kuiops for
  mm / addmm / bmm / attention / softmax / topk / gather / scatter / index / isin / cat / mean /
  all / any / max / argmax / cumsum / sort.
* ``backend`` is a ``torch.compile`` backend that lowers and then runs the FX graph as is (no
  Inductor code generation), which is enough to take the Python dispatch out of the loop.

Elementwise maps, casts, clones and masked fills are left to the compiler on purpose: fusing
them is its job.
"""
import torch
from torch.utils._pytree import tree_map

from . import registry

aten = torch.ops.aten
_LIB = None
_OPS = {}       # aten overload -> kuiops custom op (OpOverload)


# custom op name -> [calls served by a kuiops kernel, calls handed back to stock PyTorch]
call_stats = {}


def _define_same_schema(lib, name, aten_op, schema):
    """A custom op with the aten op's own signature: CUDA runs the kuiops kernel, fake runs aten.
    A graph compiled with symbolic sizes is lowered on the sizes seen at compile time; a later call
    whose actual sizes the gates refuse falls through to the aten op, as the dispatch mode does."""
    lib.define(f"{name}{schema}")
    stats = call_stats.setdefault(name, [0, 0])

    def impl(*args, **kwargs):
        out = registry.try_dispatch(aten_op, args, kwargs)
        if out is None:
            stats[1] += 1
            return aten_op(*args, **kwargs)
        stats[0] += 1
        return out
    lib.impl(name, impl, "CUDA")
    torch.library.register_fake(f"kuiops::{name}")(lambda *a, **k: aten_op(*a, **k))
    return getattr(torch.ops.kuiops, name).default


def _attention_out(q, ev, blhd):
    """Output buffer with the memory layout the replaced ATen overload would have produced, because
    the traced graph was specialised on it (a ``transpose(1, 2).contiguous().view(...)`` behind the
    attention is traced as a plain view when the transposed output is already dense): the
    efficient overload always returns (batch, row, head, dim) memory, the flash and cuDNN
    overloads return the dimension order of the query."""
    n, h, l, _ = q.shape
    if blhd:
        return q.new_empty((n, l, h, ev)).transpose(1, 2)
    order = sorted(range(3), key=lambda d: -int(q.stride(d)))            # slowest-varying first; dim 3 stays innermost
    sizes = [(n, h, l)[d] for d in order]
    buf = q.new_empty((*sizes, ev))
    return buf.permute(*[order.index(d) for d in range(3)], 3)


def _define_sdpa(lib):
    lib.define("sdpa(Tensor q, Tensor k, Tensor v, Tensor? bias, float scale, bool causal, bool blhd) -> (Tensor, Tensor)")
    stats = call_stats.setdefault("sdpa", [0, 0])

    def impl(q, k, v, bias, scale, causal, blhd):
        from . import _ffi
        stats[0] += 1
        out = _attention_out(q, v.shape[3], blhd)
        return _ffi.sdpa(q, k, v, bias=bias, scale=scale, is_causal=causal, need_lse=True, out=out)
    lib.impl("sdpa", impl, "CUDA")

    @torch.library.register_fake("kuiops::sdpa")
    def _(q, k, v, bias, scale, causal, blhd):
        out = _attention_out(q, v.shape[3], blhd)
        return out, q.new_empty((q.shape[0], q.shape[1], q.shape[2]), dtype=torch.float32)
    return torch.ops.kuiops.sdpa.default


_SCHEMAS = [
    ("mm", lambda: aten.mm.default, "(Tensor self, Tensor mat2) -> Tensor"),
    ("addmm", lambda: aten.addmm.default, "(Tensor self, Tensor mat1, Tensor mat2, *, Scalar beta=1, Scalar alpha=1) -> Tensor"),
    ("bmm", lambda: aten.bmm.default, "(Tensor self, Tensor mat2) -> Tensor"),
    ("softmax", lambda: aten._softmax.default, "(Tensor self, int dim, bool half_to_float) -> Tensor"),
    ("topk", lambda: aten.topk.default, "(Tensor self, int k, int dim=-1, bool largest=True, bool sorted=True) -> (Tensor, Tensor)"),
    ("gather", lambda: aten.gather.default, "(Tensor self, int dim, Tensor index, *, bool sparse_grad=False) -> Tensor"),
    ("scatter_src", lambda: aten.scatter.src, "(Tensor self, int dim, Tensor index, Tensor src) -> Tensor"),
    ("cat", lambda: aten.cat.default, "(Tensor[] tensors, int dim=0) -> Tensor"),
    ("index", lambda: aten.index.Tensor, "(Tensor self, Tensor?[] indices) -> Tensor"),
    ("isin", lambda: aten.isin.Tensor_Tensor, "(Tensor elements, Tensor test_elements, *, bool assume_unique=False, bool invert=False) -> Tensor"),
    ("mean_dim", lambda: aten.mean.dim, "(Tensor self, int[1]? dim, bool keepdim=False, *, ScalarType? dtype=None) -> Tensor"),
    ("all", lambda: aten.all.default, "(Tensor self) -> Tensor"),
    ("any", lambda: aten.any.default, "(Tensor self) -> Tensor"),
    ("max", lambda: aten.max.default, "(Tensor self) -> Tensor"),
    # row-wise ops of the sampling tail that a compiler does not fuse into its neighbours
    ("argmax", lambda: aten.argmax.default, "(Tensor self, int? dim=None, bool keepdim=False) -> Tensor"),
    ("cumsum", lambda: aten.cumsum.default, "(Tensor self, int dim, *, ScalarType? dtype=None) -> Tensor"),
    ("sort", lambda: aten.sort.default, "(Tensor self, int dim=-1, bool descending=False) -> (Tensor, Tensor)"),
    ("sort_stable", lambda: aten.sort.stable, "(Tensor self, *, bool? stable, int dim=-1, bool descending=False) -> (Tensor, Tensor)"),
]
_SDPA_ATEN = None


def register_ops():
    """Define the ``kuiops::*`` custom ops once per process; returns {aten overload: custom op}."""
    global _LIB, _SDPA_ATEN
    if _LIB is not None:
        return _OPS
    _LIB = torch.library.Library("kuiops", "DEF")
    for name, get, schema in _SCHEMAS:
        op = get()
        _OPS[op] = _define_same_schema(_LIB, name, op, schema)
    _OPS["sdpa"] = _define_sdpa(_LIB)
    _SDPA_ATEN = (aten._scaled_dot_product_flash_attention.default, aten._scaled_dot_product_efficient_attention.default,
                  aten._scaled_dot_product_cudnn_attention.default)
    return _OPS


_hint_mode = None


def _concrete(t):
    """A fake tensor whose sizes are symbolic -> a fake CUDA tensor with the sizes and strides seen at
    compile time (the hints), so that the gates can be asked without adding guards to the graph.
    Returns None when a size has no hint (data-dependent shapes are left to the compiler)."""
    global _hint_mode
    if not isinstance(t, torch.Tensor):
        return t
    if not any(isinstance(v, torch.SymInt) for v in tuple(t.shape) + tuple(t.stride())):
        return t
    from torch.fx.experimental.symbolic_shapes import has_hint, size_hint
    from torch._subclasses.fake_tensor import FakeTensorMode
    dims = []
    for v in tuple(t.shape) + tuple(t.stride()):
        if isinstance(v, torch.SymInt):
            if not has_hint(v):
                return None
            v = size_hint(v)
        dims.append(int(v))
    if _hint_mode is None:
        _hint_mode = FakeTensorMode()
    with _hint_mode:
        return torch.empty_strided(dims[:t.dim()], dims[t.dim():], dtype=t.dtype, device=t.device)


def _fake(x):
    return _concrete(x.meta.get("val")) if isinstance(x, torch.fx.Node) else x


def _lower_sdpa(graph, node, fam):
    """aten flash / efficient attention node -> kuiops::sdpa; only outputs 0 and 1 may be used."""
    fargs = tree_map(_fake, node.args)
    fkw = tree_map(_fake, dict(node.kwargs))
    if any(_fake(a) is None for a in node.args[:3]):
        return False
    spec = fam.supported(node.target, fargs, fkw)
    if spec is None:
        return False
    import operator
    _, scale, causal, overload, _, _ = spec
    # outputs a consumer may use: the attention output, and the log-sum-exp where its shape is (N, H, L)
    # (the cuDNN overload's is (N, H, L, 1))
    usable = (0,) if overload == "cudnn" else (0, 1)
    for user in node.users:
        if not (user.op == "call_function" and user.target is operator.getitem and user.args[1] in usable):
            if len(user.users):
                return False
    q, k, v = node.args[0], node.args[1], node.args[2]
    bias = node.args[3] if overload in ("efficient", "cudnn") else None
    with graph.inserting_before(node):
        new = graph.call_function(_OPS["sdpa"], (q, k, v, bias, float(scale), bool(causal), overload == "efficient"))
    new.meta["val"] = (node.meta["val"][0], node.meta["val"][1]) if "val" in node.meta else None
    for user in list(node.users):
        if user.target is operator.getitem and user.args[1] in (0, 1):
            user.replace_input_with(node, new)
        else:
            graph.erase_node(user)
    graph.erase_node(node)
    return True


def lower_graph(graph: torch.fx.Graph) -> int:
    """Rewrite eligible aten nodes of an aten-level FX graph in place; returns how many were
    lowered.  Eligibility is exactly ``supported()`` of the op's family under the current gates,
    evaluated on the fake tensors recorded in ``node.meta['val']``."""
    ops = register_ops()
    table = registry.table()
    lowered = 0
    for node in list(graph.nodes):
        if node.op != "call_function":
            continue
        fam = table.get(node.target)
        if fam is None:
            continue
        if node.target in _SDPA_ATEN:
            lowered += 1 if _lower_sdpa(graph, node, fam) else 0
            continue
        custom = ops.get(node.target)
        if custom is None:
            continue        # families left to the compiler (elementwise maps)
        try:
            fargs = tree_map(_fake, node.args)
            fkw = tree_map(_fake, dict(node.kwargs))
            if any(v is None for v in (_fake(a) for a in node.args if isinstance(a, torch.fx.Node))):
                continue
            spec = fam.supported(node.target, fargs, fkw)
        except Exception:
            spec = None
        if spec is None:
            continue
        node.target = custom
        lowered += 1
    graph.lint()
    return lowered


def install_inductor_pass():
    """Make Inductor run ``lower_graph`` on every post-grad graph it compiles."""
    import torch._inductor.config as icfg
    register_ops()
    icfg.post_grad_custom_post_pass = lower_graph
    return lower_graph


def backend(gm: torch.fx.GraphModule, example_inputs):
    """``torch.compile(model, backend=kuipy.inductor.backend)``: functionalise to aten, lower,
    and run the resulting FX graph (no code generation)."""
    from torch._dynamo.backends.common import aot_autograd

    def compile_fw(g, inputs):
        lower_graph(g.graph)
        g.recompile()
        return g.forward
    return aot_autograd(fw_compiler=compile_fw)(gm, example_inputs)
