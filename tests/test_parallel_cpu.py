"""Partition logic of the two multi-GPU forms, on CPU ranks (gloo, world size 2).

Tensor parallel: column-split QKV / gate / up, row-split O / down, head-sharded attention and one
all-reduce after each row-split product must reproduce the unsplit layer.  Data parallel: the
per-rank batch slices are disjoint and cover the batch.  PyTorch CPU matmuls stand in for the
kernels here; what is under test is the sharding helpers of ``kuillm_b200.decoder`` and the
collective placement."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from kuillm_b200.decoder import dp_slice, shard_in_features, shard_out_features

D, HQ, HK, HD, FF, B, S = 32, 4, 2, 8, 48, 3, 5


def _weights():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g) * 0.2
    return dict(wq=r(HQ * HD, D), wk=r(HK * HD, D), wv=r(HK * HD, D), wo=r(D, HQ * HD), wg=r(FF, D), wu=r(FF, D),
                wd=r(D, FF), x=r(B, S, D))


def _attn(q, k, v, hq, hk):
    q = q.view(B, S, hq, HD).transpose(1, 2)
    k = k.view(B, S, hk, HD).transpose(1, 2).repeat_interleave(hq // hk, 1)
    v = v.view(B, S, hk, HD).transpose(1, 2).repeat_interleave(hq // hk, 1)
    o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
    return o.transpose(1, 2).reshape(B, S, hq * HD)


def _layer(w, rank, size, reduce):
    hq, hk, ff = HQ // size, HK // size, FF // size
    x = w["x"]
    q = x @ shard_out_features(w["wq"], HQ, HD, rank, size).t()
    k = x @ shard_out_features(w["wk"], HK, HD, rank, size).t()
    v = x @ shard_out_features(w["wv"], HK, HD, rank, size).t()
    o = reduce(_attn(q, k, v, hq, hk) @ shard_in_features(w["wo"], hq * HD, rank).t())
    h = x + o
    act = F.silu(h @ shard_out_features(w["wg"], FF, 1, rank, size).t()) * (h @ shard_out_features(w["wu"], FF, 1, rank, size).t())
    return h + reduce(act @ shard_in_features(w["wd"], ff, rank).t())


def _worker(rank, size, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=size)
    calls = [0]

    def allreduce(t):
        calls[0] += 1
        dist.all_reduce(t)
        return t
    y = _layer(_weights(), rank, size, allreduce)
    ref = _layer(_weights(), 0, 1, lambda t: t)
    ok = torch.allclose(y, ref, atol=1e-5, rtol=1e-5) and calls[0] == 2      # one all-reduce per block
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        out.put(int(flag.item()))
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_tensor_parallel_layer_matches_unsplit_layer_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=10) == 1


def _lonely_worker(port, out):
    """Rank 0 of a group of two whose other rank never starts: the rendezvous must end with an error
    after its (short) timeout, on the host, and the process must stay in control."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        t = torch.ones(1)
        dist.all_reduce(t)                  # not reached with a store-based rendezvous; errors out otherwise
        out.put("joined")
    except Exception as e:                  # noqa: BLE001 - any rendezvous / collective error is the expected outcome
        out.put(f"error: {type(e).__name__}")


def test_rank_that_never_starts_is_reported_on_the_host():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_lonely_worker, args=(_free_port(), q))
    p.start()
    p.join(60)
    assert p.exitcode == 0, "the surviving rank must come back from the failed rendezvous by itself"
    assert q.get(timeout=10).startswith("error")


def test_shards_partition_the_weights():
    w = torch.arange(8 * 6.0).view(8, 6)
    parts = [shard_out_features(w, 4, 2, r, 2) for r in range(2)]          # 4 heads of 2 rows, 2 ranks
    assert torch.equal(torch.cat(parts, 0), w)
    cols = [shard_in_features(w, 3, r) for r in range(2)]
    assert torch.equal(torch.cat(cols, 1), w)


def test_data_parallel_slices_cover_the_batch_without_overlap():
    for batch, size in ((32, 8), (32, 3), (5, 8), (1, 2)):
        seen = []
        for r in range(size):
            lo, hi = dp_slice(batch, r, size)
            seen += list(range(lo, hi))
        assert seen == list(range(batch))
