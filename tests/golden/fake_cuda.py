"""A CPU tensor that answers ``is_cuda == True``.

The ``supported()`` gates only look at tensor metadata (device kind, dtype, rank, shape, numel),
so they can be exercised without a GPU by handing them such tensors.  Used by the script that
records the reference's accept / reject decisions and by the CPU tests that replay them.
"""
import torch


class FakeCudaTensor(torch.Tensor):
    @staticmethod
    def __new__(cls, data):
        return torch.Tensor._make_subclass(cls, data)

    @property
    def is_cuda(self):
        return True

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        # metadata queries only; never compute on these
        return super().__torch_function__(func, types, args, kwargs or {})


def fake(shape, dtype=torch.float32):
    if dtype in (torch.int64, torch.int32, torch.bool, torch.uint8):
        base = torch.zeros(shape, dtype=dtype)
    else:
        base = torch.zeros(shape, dtype=dtype)
    return FakeCudaTensor(base)
