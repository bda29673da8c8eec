"""Failure detection on the device side of the fused all-reduce, without any GPU fault.

``kuiops_rmsnorm_gather`` polls the stamped cells that the other ranks' GEMMs store into this
rank's receive area.  A rank that died between steps never stores its cells; the kernel must then
give up after its limit, record error word 30 and return, and the context must stay usable.  One
GPU, one process: the receive area is an ordinary buffer in which the test fills the slot of only
one of the two ranks, with the limit lowered to a millisecond through
``kuiops_debug_set_peer_wait_ns``.  Nothing here can wait past the limit."""
import time
from types import SimpleNamespace

import pytest
import torch

from kuipy import _ffi

pytestmark = pytest.mark.gpu

RANKS, ROWS, WIDTH, EPS = 2, 8, 256, 1e-5


def _area():
    slot = ROWS * WIDTH * 4                                   # 4 bytes per element: its value and half a stamp
    buf = torch.zeros(2 * RANKS * slot + 256, dtype=torch.uint8, device="cuda")
    ex = SimpleNamespace(n_ranks=RANKS, rank=0, local_base=buf.data_ptr(), slot_bytes=slot,
                         epoch=torch.zeros(1, dtype=torch.int32, device="cuda"),
                         ticket_gather=torch.zeros(1, dtype=torch.int32, device="cuda"), buffer=buf)
    cells = buf[:2 * RANKS * slot].view(torch.int32).view(2, RANKS, ROWS, WIDTH // 2, 2)     # [half][source][row][cell][(pair, stamp)]
    return ex, cells


def _deliver(cells, half, rank, part, stamp):
    """What kuiops_gemm_push stores: pairs of bf16 elements plus the stamp, cell by cell."""
    cells[half, rank, :, :, 0] = part.contiguous().view(torch.int32)
    cells[half, rank, :, :, 1] = stamp


def _expected(parts, residual, weight):
    x = sum(p.float() for p in parts).bfloat16().float()             # the all-reduce result, rounded once
    res = (x + residual.float()).bfloat16()
    rs = torch.rsqrt(res.float().pow(2).mean(-1, keepdim=True) + EPS)
    return ((res.float() * rs).bfloat16().float() * weight.float()).bfloat16(), res


def test_flag_wait_runs_out_records_30_and_the_next_call_works(cuda):
    g = torch.Generator().manual_seed(0)
    ex, cells = _area()
    weight = (1 + 0.1 * torch.randn(WIDTH, generator=g)).bfloat16().cuda()
    parts = [torch.randn(ROWS, WIDTH, generator=g).bfloat16().cuda() for _ in range(RANKS)]
    residual = torch.randn(ROWS, WIDTH, generator=g).bfloat16().cuda()
    assert _ffi.tc_error() == 0
    # exchange 0: rank 0's cells have arrived, rank 1's never do
    _deliver(cells, 0, 0, parts[0], 1)
    torch.cuda.synchronize()
    old = _ffi.set_peer_wait_ns(1_000_000)
    try:
        t0 = time.perf_counter()
        _ffi.rmsnorm_gather(ex, ROWS, weight, EPS, residual.clone())
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
    finally:
        assert _ffi.set_peer_wait_ns(old) == 1_000_000
    assert waited < 1.0, f"the kernel did not give up at its limit ({waited:.2f} s)"
    assert _ffi.tc_error() == 30 and _ffi.tc_error() == 0            # recorded once, cleared by the read
    assert int(ex.epoch.item()) == 1 and int(ex.ticket_gather.item()) == 0      # the exchange moved on, tickets are back at zero
    # exchange 1 (the other half of the area): both ranks arrive, the result is the ordinary one
    for r in range(RANKS):
        _deliver(cells, 1, r, parts[r], 2)
    res = residual.clone()
    out = _ffi.rmsnorm_gather(ex, ROWS, weight, EPS, res)
    torch.cuda.synchronize()
    want, want_res = _expected(parts, residual, weight)
    assert torch.equal(res, want_res)
    assert (out.float() - want.float()).abs().max() <= 2e-2 * want.float().abs().max()
    assert _ffi.tc_error() == 0 and int(ex.epoch.item()) == 2
