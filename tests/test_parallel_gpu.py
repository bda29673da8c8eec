"""Tensor-parallel and data-parallel decoder on two GPUs (skipped with fewer): the TP logits must
match the single-GPU logits of the same weights within the bf16 bar, with exactly two all-reduces
per layer; the fused GEMM + all-reduce form must reproduce the NCCL form bit for bit without any
NCCL call; DP ranks reproduce their slice of the single-GPU result bit for bit."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, size, port, q):
    """Child process of one rank; any exception ends the process with a non-zero code at once (the
    parent then stops the others) instead of leaving it to the collectives' time limit."""
    try:
        _tp_worker_body(rank, size, port, q)
    except BaseException:
        import traceback
        traceback.print_exc()
        os._exit(3)


def _tp_worker_body(rank, size, port, q):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    for p in (root, root / "kuillm_b200"):
        sys.path.insert(0, str(p))
    import torch.distributed as dist
    from kuillm_b200.decoder import Decoder, DecoderConfig, dp_slice
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    import datetime
    # a rank that fails leaves the others in a collective: a short limit ends them instead of the default ten minutes
    dist.init_process_group("nccl", rank=rank, world_size=size, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=180))
    cfg = DecoderConfig.tiny(n_heads=2 * size, n_kv_heads=size)
    g = torch.Generator().manual_seed(0)
    B = max(4, size)                                 # every data-parallel rank gets at least one sequence
    ids = torch.randint(0, cfg.vocab, (B, 16), generator=g).cuda()
    # reference: the whole model on this rank's GPU
    full = Decoder(cfg, device=f"cuda:{rank}", seed=0, init_std=0.05)
    full.alloc_cache(B, 24)
    ref = full.prefill(ids)
    ref_tok = ref.argmax(-1)
    ref2 = full.decode_step(ref_tok)
    # tensor parallel over the two ranks
    calls = [0]
    real = dist.all_reduce

    def counted(t, *a, **k):
        calls[0] += 1
        return real(t, *a, **k)
    dist.all_reduce = counted
    tp = Decoder(cfg, device=f"cuda:{rank}", seed=0, init_std=0.05, tp_rank=rank, tp_size=size)
    tp.alloc_cache(B, 24)
    out = tp.prefill(ids)
    n_calls = calls[0]
    out2 = tp.decode_step(ref_tok)
    dist.all_reduce = real
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    # vocabulary-parallel greedy step: best (value, id) pairs exchanged instead of the logits; ties go to the lowest id
    from kuipy import _ffi as _f
    per = cfg.vocab // size
    tok_tp = tp.next_token(out2[:, rank * per:(rank + 1) * per].contiguous())
    ok_tok = torch.equal(tok_tp, _f.argmax_lastdim(out2))
    ok_tp = rel(out, ref) < 3e-2 and rel(out2, ref2) < 3e-2 and n_calls == 2 * cfg.n_layers and ok_tok
    # the same prefill with its all-reduces hidden behind the other half of the batch: same logits (the sums are
    # element-wise, whatever the message size), same caches (the next decode step agrees), twice the calls
    tpo = Decoder(cfg, device=f"cuda:{rank}", seed=0, init_std=0.05, tp_rank=rank, tp_size=size)
    tpo.alloc_cache(B, 24)
    tpo.overlap_min_rows = 1
    calls[0] = 0
    dist.all_reduce = counted
    outo = tpo.prefill(ids)
    n_over = calls[0]
    dist.all_reduce = real
    outo2 = tpo.decode_step(ref_tok)
    ok_tp = ok_tp and rel(outo, out) < 1e-2 and rel(outo2, out2) < 1e-2 and n_over == 4 * cfg.n_layers
    # the fused form: row-split GEMMs push their partials into both ranks' memory, the next norm sums
    # them; no NCCL call on that path, and with two ranks the sum rounds exactly as NCCL's does
    from kuipy import _ffi
    tpf = Decoder(cfg, device=f"cuda:{rank}", seed=0, init_std=0.05, tp_rank=rank, tp_size=size)
    tpf.alloc_cache(B, 24)
    tpf.enable_fused_allreduce(128)
    calls[0] = 0
    dist.all_reduce = counted
    f1 = tpf.prefill(ids)                     # 64 rows (128 with eight ranks): small enough for the fused path
    tok = ref_tok
    # two ranks: fp32 sum of two rounded partials, rounded once, is what NCCL computes too; with more
    # ranks NCCL's order of additions is its own, so the forms agree only within rounding
    agree = (lambda a, bq: torch.equal(a, bq)) if size == 2 else (lambda a, bq: rel(a, bq) < 1e-2)
    same = agree(f1, out)
    worst = rel(f1, ref)
    tp.length = tpf.length                    # the NCCL decoder took one decode step above: rewind it
    for _ in range(5):
        a, bq = tp.decode_step(tok), tpf.decode_step(tok)
        same = same and agree(a, bq)
        tok = a.argmax(-1)
    fused_calls = calls[0] - 5 * 2 * cfg.n_layers      # the NCCL decoder's own calls in the loop
    dist.all_reduce = real
    torch.cuda.synchronize()
    ok_fused = same and worst < 3e-2 and fused_calls == 0 and _ffi.tc_error() == 0 and int(tpf.exchange.epoch.item()) == 6 * 2 * cfg.n_layers
    ok_tp = ok_tp and ok_fused
    # data parallel: this rank's slice of the batch, no collective
    lo, hi = dp_slice(B, rank, size)
    dp = Decoder(cfg, device=f"cuda:{rank}", seed=0, init_std=0.05)
    dp.alloc_cache(hi - lo, 24)
    ok_dp = torch.equal(dp.prefill(ids[lo:hi]), ref[lo:hi])
    flag = torch.tensor([1 if (ok_tp and ok_dp) else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        q.put((int(flag.item()), rel(out, ref), rel(out2, ref2), n_calls, bool(ok_fused), bool(same), fused_calls))
    dist.destroy_process_group()


@pytest.mark.parametrize("size", [2, 4, 8])
def test_tp_and_dp_match_single_gpu(size):
    if not torch.cuda.is_available() or torch.cuda.device_count() < size:
        pytest.skip(f"needs {size} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, size, port, q)) for r in range(size)]
    for p in procs:
        p.start()
    import time
    deadline = time.time() + 300
    while time.time() < deadline and any(p.exitcode is None for p in procs) and not any(p.exitcode not in (None, 0) for p in procs):
        time.sleep(0.5)
    codes = [p.exitcode for p in procs]
    for p in procs:                                   # a failed or late rank: stop exactly the children started here
        if p.exitcode is None:
            p.kill()
        p.join(10)
    assert codes == [0] * size, codes
    ok, r1, r2, n, ok_fused, same, fused_calls = q.get(timeout=10)
    assert ok == 1, (r1, r2, n, ok_fused, same, fused_calls)
