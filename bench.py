"""Decode + prefill throughput of the kuiops library on a Llama-3-8B-shaped decoder.

    python bench.py --gpus N --steps K --warmup W            # this library (one rank per GPU)
    python bench.py --impl reference --gpus N ...           # the reference's CPU path (rank 0 only)

A step is one greedy generation over one batch of synthetic prompts: prefill of 32 x 2048
uniform-random token ids, then 256 decoded tokens per sequence (random-init N(0, 0.02) bf16
weights of the 8B shape; no dataset, no checkpoint).  ``value`` is generated tokens per second
over the whole call, prefill included - the number the reference prints (infer.py:159-166
there) - summed over ranks; ``config`` carries the prefill / decode split measured the way
infer_minimal.py:68-76 does.  With N > 1 every rank runs its own batch of 32 (batch data
parallel, no collective, weak scaling); ``--parallel tp`` runs the tensor-parallel form on one
global batch instead.

Timing: W warm-up steps, then exactly K steps between barrier + synchronize, CUDA events on the
launching stream, max over ranks.  The 15 GB of weights streamed per decode step exceed the
126 MB L2, so no flush is needed between iterations.  GPU clocks and throttle reasons are
sampled with nvidia-smi during the timed region.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "kuillm_b200"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

WORKLOADS = {
    # name: (decoder config kwargs or None for the 8B shape, batch, prompt, new tokens)
    "llama3-8b-shaped b32 p2048 d256": (None, 32, 2048, 256),
    "tiny-llama-shaped b4 p64 d8": (dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=512, vocab=1000), 4, 64, 8),
}
DEFAULT_WORKLOAD = "llama3-8b-shaped b32 p2048 d256"
# bytes per launch of gemm_tc_kernel with the SwiGLU epilogue at M=32, N=28672, K=4096 (bf16), from ncu
NCU_TRAFFIC_GATEUP_M32 = 240.1e6


class ClockSampler:
    """nvidia-smi clocks / throttle reasons for one GPU, every 200 ms, while running."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_peaks():
    try:
        return json.loads((ROOT / "MEASURED_PEAKS.json").read_text()), "measured"
    except (OSError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ---------------------------------------------------------------------------------------------
# the reference arm: the reference's CPU path = stock PyTorch eager generation on host cores
# ---------------------------------------------------------------------------------------------
def cpu_reference_sample(workload):
    """Time torch-eager greedy generation (the reference with Kuiper off, infer.py:135-148) of a
    Llama-shaped model on the host CPU, on a bounded sample of the workload: the same layer
    dimensions and vocabulary, but 1 and 2 layers, a small batch and a short prompt.  The two
    layer counts separate the per-layer cost from the fixed cost (embedding, vocabulary GEMM), so
    the extrapolation to the full depth does not multiply the fixed part; batch and prompt scale
    linearly.  Returns (tok_per_s at the full workload's shape, description, threads)."""
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg_kw, batch, prompt, new = WORKLOADS[workload]
    full = dict(n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, d_ff=14336, vocab=128256)
    if cfg_kw:
        full.update(cfg_kw)
    threads = torch.get_num_threads()
    s_batch, s_prompt, s_new = min(batch, 4), min(prompt, 256), min(new, 8)
    hf = LlamaConfig(hidden_size=full["d_model"], intermediate_size=full["d_ff"], num_hidden_layers=2,
                     num_attention_heads=full["n_heads"], num_key_value_heads=full["n_kv_heads"], head_dim=full["head_dim"],
                     vocab_size=full["vocab"], rms_norm_eps=1e-5, rope_theta=5e5, max_position_embeddings=8192,
                     tie_word_embeddings=False)
    torch.manual_seed(0)
    model = LlamaForCausalLM(hf).eval()
    ids = torch.randint(0, full["vocab"], (s_batch, s_prompt))
    ids_short = ids[:, :16]                            # decode steps are timed behind a short prompt, so that
    s_new = max(s_new, 2)                              # the prefill's run-to-run noise does not swamp them

    def timed(inp, n_new):
        t0 = time.perf_counter()
        with torch.no_grad():
            model.generate(inp, max_new_tokens=n_new, min_new_tokens=n_new, do_sample=False, pad_token_id=0)
        return time.perf_counter() - t0

    pre, dec = {}, {}
    for layers in (1, 2):
        model.config.num_hidden_layers = layers        # the model walks layers[:num_hidden_layers]
        timed(ids, 1)                                  # warm-up
        pre[layers] = min(timed(ids, 1), timed(ids, 1))      # prefill = time to the first token (infer_minimal.py:68-69)
        first = min(timed(ids_short, 1), timed(ids_short, 1))
        dec[layers] = max(timed(ids_short, s_new) - first, 1e-9) / (s_new - 1)
    # t(L) = fixed + per_layer * L
    pre_layer, dec_layer = max(pre[2] - pre[1], 0.0), max(dec[2] - dec[1], 0.0)
    pre_fixed, dec_fixed = max(pre[1] - pre_layer, 0.0), max(dec[1] - dec_layer, 0.0)
    L = full["n_layers"]
    t_prefill_full = (pre_fixed + pre_layer * L) * (prompt / s_prompt) * (batch / s_batch)
    t_decode_full = (dec_fixed + dec_layer * L) * (batch / s_batch) * (new - 1)
    tok_s = batch * new / (t_prefill_full + t_decode_full)
    desc = (f"torch eager fp32 on CPU, HF LlamaForCausalLM with the workload's layer dims and vocabulary, 1 and 2 of "
            f"{L} layers, batch {s_batch}, prompt {s_prompt}, {s_new} new tokens; measured per layer: prefill "
            f"{pre_layer:.2f}s, decode step {dec_layer * 1e3:.0f} ms; fixed part: prefill {pre_fixed:.2f}s, decode step "
            f"{dec_fixed * 1e3:.0f} ms; extrapolated linearly in layers, batch and tokens (attention's quadratic term "
            f"ignored, which favours the CPU)")
    return tok_s, desc, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    desc, threads = "", 1
    for _ in range(max(1, min(args.steps, 2))):
        v, desc, threads = cpu_reference_sample(args.workload)
        vals.append(v)
    v = sorted(vals)[len(vals) // 2]
    cfg_kw, batch, prompt, new = WORKLOADS[args.workload]
    replicas = 1 if args.parallel == "tp" else max(1, args.gpus)
    line = {"impl": "reference", "metric": "decode+prefill tok/s", "value": v, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": batch * replicas * new / v * 1e3, "higher_is_better": True,
            "scaling": "strong" if args.parallel == "tp" else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            # the same workload as this library's arm at --gpus N: N replicas of the batch (weak scaling); the host's
            # rate in tok/s does not depend on how many replicas are queued, only the time per step does
            "config": {"workload": args.workload, "global_batch": batch * replicas, "prompt_len": prompt, "new_tokens": new,
                       "parallelism": "cpu"},
            "cpu_baseline": {"value": v, "unit": "tok/s", "cores": threads, "kind": "port", "sample": desc},
            "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# this library
# ---------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    from kuipy import _ffi
    from kuillm_b200.decoder import Decoder, DecoderConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kuiops kernels have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    tp = world if args.parallel == "tp" else 1

    cfg_kw, batch, prompt, new = WORKLOADS[args.workload]
    cfg = DecoderConfig(**cfg_kw) if cfg_kw else DecoderConfig.llama3_8b()
    dec = Decoder(cfg, device=dev, seed=0, tp_rank=rank if tp > 1 else 0, tp_size=tp)
    dec.alloc_cache(batch, prompt + new)
    fused = tp > 1 and args.allreduce == "fused"
    fused_note = ""
    if fused:
        # decode steps only (batch rows); the prefill keeps NCCL.  The fused form needs every rank's
        # receive area mapped into every process; where that cannot be had the step keeps NCCL, and says so
        import torch.distributed as dist
        try:
            dec.enable_fused_allreduce(batch)
            ok = torch.ones(1, device=dev)
        except Exception as e:            # noqa: BLE001 - whatever the mapping raised is reported, not hidden
            fused_note = f"{type(e).__name__}: {e}"[:160]
            ok = torch.zeros(1, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            dec.exchange, fused = None, False
            if rank == 0:
                print(f"[bench] fused all-reduce unavailable, using NCCL: {fused_note or 'another rank failed'}", file=sys.stderr)
    g = torch.Generator().manual_seed(1000 + (0 if tp > 1 else rank))
    ids_host = torch.randint(0, cfg.vocab, (batch, prompt), generator=g).pin_memory()
    ids_dev = ids_host.to(dev)
    out_host = torch.empty((batch, new), dtype=torch.int64).pin_memory()

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    ev = lambda: torch.cuda.Event(enable_timing=True)

    use_graph = not args.no_graph
    if use_graph:
        dec.capture_decode(batch)
    gen_buf = torch.empty((batch, new), dtype=torch.int64, device=dev)
    replays = [0]

    def one_step(ids, marks=None):
        """One generation: prefill, first token, then new - 1 decode steps (captured in a CUDA
        graph unless --no-graph).  Returns the [batch, new] generated ids (a device buffer)."""
        dec.length = 0
        if marks is not None:
            marks[0].record()
        logits = dec.prefill(ids)
        tok = _ffi.argmax_lastdim(logits)
        gen_buf[:, 0].copy_(tok)
        if marks is not None:
            marks[1].record()
        if use_graph:
            dec.decode_graph(tok, new - 1, out=gen_buf[:, 1:])
            replays[0] += new - 1
        else:
            for t in range(1, new):
                tok = _ffi.argmax_lastdim(dec.decode_step(tok))
                gen_buf[:, t].copy_(tok)
        if marks is not None:
            marks[2].record()
        return gen_buf

    for _ in range(args.warmup):
        one_step(ids_dev)
    barrier()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    marks = [[ev(), ev(), ev()] for _ in range(args.steps)]
    n0 = _ffi.launch_count()
    replays[0] = 0
    barrier()
    t_start, t_end = ev(), ev()
    t_start.record()
    for s in range(args.steps):
        one_step(ids_dev, marks[s])
    t_end.record()
    barrier()
    launches = _ffi.launch_count() - n0 + (replays[0] * dec.graph_launches if use_graph else 0)
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t_start.elapsed_time(t_end)
    prefill_ms = sum(m[0].elapsed_time(m[1]) for m in marks) / args.steps
    decode_ms = sum(m[1].elapsed_time(m[2]) for m in marks) / args.steps

    # end to end through the public call with host buffers: pinned ids in, generated ids out
    barrier()
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(args.steps):
        ids_in = ids_host.to(dev, non_blocking=True)
        out_host.copy_(one_step(ids_in), non_blocking=True)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)

    if _ffi.tc_error() != 0:
        raise SystemExit("a tensor-core pipeline wait timed out during the bench; numbers discarded")

    # roofline of the dominant decode kernel: the gate|up weight-streaming GEMM with its fused SwiGLU
    # epilogue, exactly the launch the decode step makes, timed live over the 32 layers' distinct
    # weights (7.5 GB, far beyond L2): the 32 launches are replayed from a CUDA graph, as in the
    # decode step, with events on the replaying stream
    x = torch.randn(batch, cfg.d_model, device=dev).to(cfg.dtype)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for L in dec.layers[:3]:
            _ffi.gemm_swiglu(x, L["wgu"])
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for L in dec.layers:
                _ffi.gemm_swiglu(x, L["wgu"])
        g.replay()
        side.synchronize()
        r0, r1 = ev(), ev()
        r0.record(side)
        g.replay()
        r1.record(side)
        side.synchronize()
    torch.cuda.current_stream(dev).wait_stream(side)
    gemm_ms = r0.elapsed_time(r1) / len(dec.layers)
    del g
    n_out, k_in = dec.layers[0]["wgu"].shape
    alg_bytes = 2 * (n_out * k_in + batch * k_in + batch * n_out // 2)
    peaks, peak_kind = measured_peaks()
    achieved = alg_bytes / (gemm_ms * 1e-3) / 1e9
    # DRAM bytes one such launch moved under ncu (dram__bytes_read.sum + dram__bytes_write.sum of the
    # capture summarised in profiles/ncu_gemm_m32_gateup.md); only meaningful for the full-size weights
    traffic = NCU_TRAFFIC_GATEUP_M32 if (n_out, k_in, batch, tp) == (28672, 4096, 32, 1) else None

    vals = torch.tensor([total_ms, e2e_ms, prefill_ms, decode_ms], device=dev, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, prefill_ms, decode_ms = vals.tolist()
    replicas = 1 if tp > 1 else world
    gen_tokens = batch * new * replicas * args.steps
    value = gen_tokens / (total_ms * 1e-3)

    if rank == 0:
        line = {
            "metric": "decode+prefill tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if tp > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "global_batch": batch * replicas, "prompt_len": prompt, "new_tokens": new,
                       "parallelism": (f"tp{tp}" if tp > 1 else f"dp{world}"), "decode_cuda_graph": use_graph,
                       **({"decode_allreduce": "fused into the GEMM epilogue and the next norm (peer stores)" if fused else "nccl"} if tp > 1 else {}),
                       "prefill_tok_s": batch * prompt * replicas / (prefill_ms * 1e-3),
                       "decode_tok_s": batch * (new - 1) * replicas / (decode_ms * 1e-3),
                       "prefill_ms": prefill_ms, "decode_ms_per_token": decode_ms / (new - 1),
                       "l2": "weights streamed per step (15 GB at the 8B shape) exceed the 126 MB L2; no flush"},
            "e2e": {"value": gen_tokens / (e2e_ms * 1e-3), "unit": "tok/s",
                    "h2d_bytes_per_step": ids_host.numel() * 8, "d2h_bytes_per_step": out_host.numel() * 8},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"kernel": "gemm_tc_kernel (gate|up projection + SwiGLU epilogue of one decode step)", "bound": "hbm",
                         "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "peak_kind": peak_kind, "nominal_peak": 8000.0, "frac_nominal": achieved / 8000.0,
                         "traffic": traffic, "us_per_launch": gemm_ms * 1e3,
                         "algorithmic_bytes_per_launch": alg_bytes},
        }
        if world == 1 and not args.no_cpu_baseline:
            v, desc, threads = cpu_reference_sample(args.workload)
            line["cpu_baseline"] = {"value": v, "unit": "tok/s", "cores": threads, "kind": "port", "sample": desc}
        print(json.dumps(line))
    if world > 1:
        # a captured graph may hold NCCL work: drop it and drain the device before the ranks part,
        # then leave without tearing the communicator down (teardown after graph capture can block)
        import torch.distributed as dist
        dec._graph = None
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--parallel", default="dp", choices=["dp", "tp"])
    ap.add_argument("--allreduce", default="fused", choices=["fused", "nccl"],
                    help="tensor parallel only: how the decode step sums the row-split projections")
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=list(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every decode kernel from the host instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
