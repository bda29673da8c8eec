"""Receive areas of a tensor-parallel group, mapped into every rank: the memory behind the fused
row-split GEMM + all-reduce of the decode step (``kuiops_gemm_push`` / ``kuiops_rmsnorm_gather``).

Each rank owns one symmetric allocation laid out as

    [2 halves][n_ranks sources][slot_bytes]   partial products, one slot per (epoch parity, source),

a slot being rows x width / 2 cells of 8 bytes: two 16-bit elements and the 32-bit stamp epoch + 1
(a cell is valid as soon as it is seen with the expected stamp: no flags, no fences).  The rank holds the device address of every rank's allocation (``torch.distributed._symmetric_memory``
does the handle exchange).  Pushes are plain stores through those peer addresses over NVLink; no
multicast object is bound (it is switched off before the first rendezvous).
"""
import ctypes
import os

import torch


class PeerExchange:
    def __init__(self, group, device, max_rows, width, dtype):
        import torch.distributed as dist
        # assigned, not defaulted: an inherited "0" would let the rendezvous bind an NVLink multicast object
        os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
        import torch.distributed._symmetric_memory as symm
        if group is None:
            group = dist.group.WORLD
        self.n_ranks = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if torch.empty((), dtype=dtype).element_size() != 2:
            raise ValueError("kuiops: the exchange cells hold 16-bit elements")
        self.slot_bytes = (max_rows * width * 4 + 255) // 256 * 256
        total = 2 * self.n_ranks * self.slot_bytes + 256
        self.buffer = symm.empty(total, dtype=torch.uint8, device=device)
        self.buffer.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm.rendezvous(self.buffer, group)
        if int(getattr(self.handle, "multicast_ptr", 0) or 0) != 0:
            raise RuntimeError("kuiops: the symmetric-memory rendezvous bound a multicast object; the fused "
                               "all-reduce only runs on plain peer mappings")
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(ptrs) != self.n_ranks or ptrs[self.rank] != self.buffer.data_ptr():
            raise RuntimeError("kuiops: symmetric memory rendezvous returned unexpected addresses")
        self.peer_array = (ctypes.c_uint64 * self.n_ranks)(*ptrs)
        self.local_base = self.buffer.data_ptr()
        # device words: the exchange counter and the gathering kernel's ticket
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.ticket_gather = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)          # nobody pushes before every area is zeroed and mapped
