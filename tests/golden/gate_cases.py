"""The matrix of calls whose accept / reject decision is recorded from the reference gates.

Each case is (family class name, aten overload name, positional argument descriptors, kwargs).
A descriptor is ``("T", shape, dtype_name)`` for a (fake CUDA) tensor, ``("CPU", shape,
dtype_name)`` for a real CPU tensor, ``("L", [descriptors])`` for a list, or a plain Python
value.  Shared by the generating script (run against the reference) and the CPU test (run
against this repository), so both see identical inputs.
"""
import itertools

import torch

DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16, "f64": torch.float64,
      "i64": torch.int64, "i32": torch.int32, "bool": torch.bool, "u8": torch.uint8}


def T(shape, dt="f32"):
    return ("T", list(shape), dt)


def cases():
    out = []
    add = out.append
    # ---- mm: tile divisibility decides in the reference ------------------------------------
    mm_shapes = [(64, 64, 64), (128, 64, 128), (128, 63, 128), (32, 32, 32), (16, 4096, 4096), (1, 4096, 4096),
                 (8, 64, 64), (4096, 4096, 4096), (128, 14336, 4096), (96, 64, 64), (64, 48, 64), (64, 64, 16),
                 (64, 64, 8), (256, 128, 32), (17, 9, 13), (128, 128256, 4096), (64, 96, 64), (192, 192, 192)]
    for (M, N, K), dt in itertools.product(mm_shapes, ("f32", "bf16", "f16")):
        add(("MmImpl", "mm.default", [T((M, K), dt), T((K, N), dt)], {}))
    add(("MmImpl", "mm.default", [T((64, 64)), T((32, 64))], {}))                 # K mismatch
    add(("MmImpl", "mm.default", [T((64, 64)), T((64, 64), "bf16")], {}))         # dtype mismatch
    add(("MmImpl", "mm.default", [T((2, 64, 64)), T((64, 64))], {}))              # rank
    add(("MmImpl", "mm.default", [("CPU", [64, 64], "f32"), ("CPU", [64, 64], "f32")], {}))
    # ---- bmm --------------------------------------------------------------------------------
    for dt in ("f32", "bf16", "f16"):
        add(("BmmImpl", "bmm.default", [T((5, 17, 9), dt), T((5, 9, 13), dt)], {}))
        add(("BmmImpl", "bmm.default", [T((32, 4096, 128), dt), T((32, 128, 4096), dt)], {}))
    add(("BmmImpl", "bmm.default", [T((2, 4, 4)), T((3, 4, 4))], {}))
    add(("BmmImpl", "bmm.default", [T((4, 4)), T((4, 4))], {}))
    add(("BmmImpl", "bmm.default", [T((2, 4, 5)), T((2, 4, 4))], {}))
    add(("BmmImpl", "bmm.default", [T((2, 4, 4)), T((2, 4, 4), "bf16")], {}))
    add(("BmmImpl", "bmm.default", [T((1, 65536, 8)), T((1, 8, 65536))], {}))     # M*N beyond the launch limit
    # ---- addmm ------------------------------------------------------------------------------
    for dt in ("f32", "bf16", "f16"):
        for ab in ({}, {"alpha": 0.5, "beta": 2.0}):
            add(("AddmmImpl", "addmm.default", [T((64, 64), dt), T((64, 64), dt), T((64, 64), dt)], dict(ab)))
    add(("AddmmImpl", "addmm.default", [T((32, 32), "f64"), T((32, 32), "f64"), T((32, 32), "f64")], {}))
    add(("AddmmImpl", "addmm.default", [T((32,)), T((32, 32)), T((32, 32))], {}))          # 1-D bias
    add(("AddmmImpl", "addmm.default", [T((1, 32)), T((32, 32)), T((32, 32))], {}))        # [1, N] bias
    add(("AddmmImpl", "addmm.default", [T((32, 32)), T((32, 31)), T((31, 32))], {}))       # no tile for K = 31
    add(("AddmmImpl", "addmm.default", [T((4096, 4096), "bf16"), T((4096, 4096), "bf16"), T((4096, 4096), "bf16")], {}))
    add(("AddmmImpl", "addmm.default", [T((64, 64)), T((64, 64)), T((32, 64))], {}))
    # ---- softmax ----------------------------------------------------------------------------
    for shape, dt in itertools.product([(128, 64), (8, 5, 33), (64, 128256), (7,)], ("f32", "bf16", "f16")):
        add(("SoftmaxImpl", "_softmax.default", [T(shape, dt), len(shape) - 1, False], {}))
        add(("SoftmaxImpl", "_softmax.default", [T(shape, dt), -1, False], {}))
    add(("SoftmaxImpl", "_softmax.default", [T((16, 16)), 0, False], {}))
    add(("SoftmaxImpl", "_softmax.default", [T((16, 16)), 1, True], {}))
    add(("SoftmaxImpl", "_softmax.default", [T((16, 16), "i64"), 1, False], {}))
    # ---- mean -------------------------------------------------------------------------------
    for shape, dt in itertools.product([(4, 16), (2, 3, 4096), (32, 2048, 4096)], ("f32", "bf16")):
        add(("MeanImpl", "mean.dim", [T(shape, dt), [-1], True], {}))
        add(("MeanImpl", "mean.dim", [T(shape, dt), [len(shape) - 1], True], {}))
        add(("MeanImpl", "mean.dim", [T(shape, dt), [0], True], {}))
        add(("MeanImpl", "mean.dim", [T(shape, dt), [-1], False], {}))
        add(("MeanImpl", "mean.dim", [T(shape, dt), [-1], True], {"dtype": torch.float32}))
    add(("MeanImpl", "mean.dim", [T((4, 4, 4)), [0, 1], True], {}))
    add(("MeanImpl", "mean.dim", [T((4, 4), "i64"), [-1], True], {}))
    # ---- gather -----------------------------------------------------------------------------
    for dt in ("f32", "bf16", "i64", "bool"):
        add(("GatherImpl", "gather.default", [T((8, 5), dt), 1, T((8, 4), "i64")], {}))
        add(("GatherImpl", "gather.default", [T((8, 5), dt), 0, T((7, 5), "i64")], {}))
        add(("GatherImpl", "gather.default", [T((4, 3, 6), dt), 2, T((4, 3, 5), "i64")], {}))
        add(("GatherImpl", "gather.default", [T((4, 3, 6), dt), -1, T((4, 3, 6), "i64")], {}))
    add(("GatherImpl", "gather.default", [T((64, 2048), "i64"), 1, T((64, 2048), "i64")], {}))
    add(("GatherImpl", "gather.default", [T((4, 4)), 1, T((4, 4), "i32")], {}))
    add(("GatherImpl", "gather.default", [T((4, 4)), 1, T((4,), "i64")], {}))
    add(("GatherImpl", "gather.default", [T((4, 4)), 1, T((4, 5), "i64")], {}))          # larger on the gathered axis
    add(("GatherImpl", "gather.default", [T((4, 4)), 1, T((5, 4), "i64")], {}))          # larger off the gathered axis
    add(("GatherImpl", "gather.default", [T((4, 4)), 1, T((4, 4), "i64")], {"sparse_grad": True}))
    # ---- scatter ----------------------------------------------------------------------------
    for dt in ("f32", "bf16", "i64", "bool"):
        add(("ScatterImpl", "scatter.src", [T((8, 5), dt), 1, T((8, 5), "i64"), T((8, 5), dt)], {}))
        add(("ScatterImpl", "scatter.src", [T((8, 5), dt), 0, T((6, 5), "i64"), T((6, 5), dt)], {}))
        add(("ScatterImpl", "scatter.src", [T((4, 3, 6), dt), 2, T((4, 3, 6), "i64"), T((4, 3, 6), dt)], {}))
    add(("ScatterImpl", "scatter.src", [T((4, 4)), 1, T((4, 4), "i64"), T((4, 4), "bf16")], {}))
    add(("ScatterImpl", "scatter.src", [T((4, 4)), 1, T((4, 4), "i32"), T((4, 4))], {}))
    add(("ScatterImpl", "scatter.src", [T((4, 4)), 1, T((4, 4), "i64"), T((4, 5))], {}))
    add(("ScatterImpl", "scatter.src", [T((4, 4)), 1, T((5, 4), "i64"), T((5, 4))], {}))
    # ---- cat --------------------------------------------------------------------------------
    for dt, dim in itertools.product(("f32", "bf16", "i64"), (0, 1, 2)):
        b = [4, 3, 6]
        b[dim] += 2
        add(("CatImpl", "cat.default", [("L", [T((4, 3, 6), dt), T(b, dt)]), dim], {}))
    add(("CatImpl", "cat.default", [("L", [T((4, 4)), T((4, 4)), T((4, 4))]), 0], {}))    # 3 inputs
    add(("CatImpl", "cat.default", [("L", [T((64, 512), "i64")] * 8), 1], {}))             # 8 inputs
    add(("CatImpl", "cat.default", [("L", [T((4, 4)), T((4, 5))]), 0], {}))
    add(("CatImpl", "cat.default", [("L", [T((4, 4)), T((4, 4), "bf16")]), 0], {}))
    add(("CatImpl", "cat.default", [("L", [T((4, 4)), T((4, 4))]), -1], {}))
    add(("CatImpl", "cat.default", [("L", [T((4, 4)), T((4, 4))])], {}))
    # ---- elementwise ------------------------------------------------------------------------
    unary = ["silu.default", "neg.default", "rsqrt.default", "cos.default", "sin.default", "bitwise_not.default"]
    for op, dt in itertools.product(unary, ("f32", "bf16", "f16", "bool", "i64")):
        add(("ElementwiseImpl", op, [T((3, 5, 7), dt)], {}))
    binary = ["add.Tensor", "mul.Tensor", "sub.Tensor", "div.Tensor", "bitwise_and.Tensor", "bitwise_or.Tensor"]
    for op, dt in itertools.product(binary, ("f32", "bf16", "bool", "i64")):
        add(("ElementwiseImpl", op, [T((3, 5, 7), dt), T((3, 5, 7), dt)], {}))
        add(("ElementwiseImpl", op, [T((3, 5, 7), dt), T((5, 7), dt)], {}))              # broadcasting
    for op in ("add.Tensor", "sub.Tensor", "mul.Tensor", "div.Tensor", "add.Scalar", "mul.Scalar", "sub.Scalar",
               "div.Scalar", "pow.Tensor_Scalar"):
        add(("ElementwiseImpl", op, [T((4, 9)), 1.5], {}))
        add(("ElementwiseImpl", op, [T((4, 9), "bf16"), 2], {}))
    add(("ElementwiseImpl", "add.Tensor", [T((4, 9)), T((4, 9))], {"alpha": 2}))
    add(("ElementwiseImpl", "pow.Tensor_Scalar", [T((4, 9)), 2], {}))
    for op in ("eq.Scalar", "le.Scalar", "lt.Scalar"):
        add(("ElementwiseImpl", op, [T((5, 8)), 0.5], {}))
        add(("ElementwiseImpl", op, [T((5, 8), "i64"), 1], {}))
    add(("ElementwiseImpl", "le.Tensor", [T((4, 4)), T((4, 4))], {}))
    add(("ElementwiseImpl", "lt.Tensor", [T((4, 4)), T((4, 4))], {}))
    add(("ElementwiseImpl", "where.self", [T((3, 4, 5), "bool"), T((3, 4, 5)), T((3, 4, 5))], {}))
    add(("ElementwiseImpl", "where.self", [T((3, 4, 5), "bool"), T((3, 4, 5), "bf16"), T((3, 4, 5), "bf16")], {}))
    add(("ElementwiseImpl", "where.self", [T((4, 4), "bool"), T((4, 4)), T((4, 3))], {}))
    add(("ElementwiseImpl", "where.self", [T((4, 4), "bool"), T((4, 4)), T((4, 4), "bf16")], {}))
    add(("ElementwiseImpl", "where.self", [T((4, 4), "f32"), T((4, 4)), T((4, 4))], {}))
    # ---- sdpa (efficient-attention overload; written but unconnected in the reference) --------
    q = lambda dt: [T((2, 3, 8, 16), dt), T((2, 3, 10, 16), dt), T((2, 3, 10, 12), dt), T((2, 3, 8, 10), dt), True]
    for dt in ("f32", "bf16"):
        add(("SdpaImpl", "_scaled_dot_product_efficient_attention.default", q(dt), {"scale": 0.3}))
        add(("SdpaImpl", "_scaled_dot_product_efficient_attention.default", q(dt), {}))
        add(("SdpaImpl", "_scaled_dot_product_efficient_attention.default", q(dt) + [0.0, True], {}))
        add(("SdpaImpl", "_scaled_dot_product_efficient_attention.default", q(dt) + [0.1, False], {}))
    add(("SdpaImpl", "_scaled_dot_product_efficient_attention.default",
         [T((2, 3, 8, 16)), T((2, 3, 10, 16)), T((2, 3, 10, 12)), None, True], {}))
    add(("SdpaImpl", "_scaled_dot_product_efficient_attention.default",
         [T((2, 4, 8, 16)), T((2, 2, 10, 16)), T((2, 2, 10, 12)), T((2, 4, 8, 10)), True], {}))   # GQA
    return out
