"""Decode + prefill throughput of the kuiops library on a Llama-3-8B-shaped decoder.

    python bench.py --gpus N --steps K --warmup W            # this library (one rank per GPU)
    python bench.py --impl reference --gpus N ...           # the reference's CPU path (rank 0 only)

A step is one greedy generation over one batch of synthetic prompts: prefill of 32 x 2048
uniform-random token ids, then 256 decoded tokens per sequence (random-init N(0, 0.02) bf16
weights of the 8B shape; no dataset, no checkpoint).  ``value`` is generated tokens per second
over the whole call, prefill included - the number the reference prints (infer.py:159-166
there) - summed over ranks; ``detail`` carries the prefill / decode split measured the way
infer_minimal.py:68-76 does.  With N > 1 every rank runs its own batch of 32 (batch data
parallel, no collective, weak scaling) and, after that, the ranks together run the
tensor-parallel form on one global batch of 32 (``tp`` in the line; strong scaling).

The line also carries, measured in the same run on rank 0 at N = 1:
  * ``e2e``      the same generation through the C ABI with host buffers (pinned ids in, ids out);
  * ``plugin``   a HuggingFace Llama of the same shape generating under ``kuipy.KuiperMode()`` (the
                 reference's timed region, infer.py:135-148 there) and with its forward compiled by
                 ``torch.compile(backend=kuipy.inductor.backend)``: what a drop-in user gets, Python
                 dispatch included;
  * ``configs0`` the reference's own CPU-runnable case (GPT-2-small shape, fp32, batch 1, prompt 128,
                 64 new tokens): really timed on the host cores with the kernels off, and on the GPU
                 under ``KuiperMode``;
  * ``op_table`` the attention / GEMM / sampling operator sweeps as fractions of the measured peaks;
  * ``roofline`` of the dominant decode kernel and ``cpu_baseline`` (a bounded sample of the workload
                 on the host cores).

Timing: W warm-up steps, then exactly K steps between barrier + synchronize, CUDA events on the
launching stream, max over ranks.  The 15 GB of weights streamed per decode step exceed the
126 MB L2, so no flush is needed between iterations.  GPU clocks and throttle reasons are
sampled with nvidia-smi during the timed region.
"""
import argparse
import gc
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
    "tiny-llama-shaped b4 p64 d8": (dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=128, d_ff=512, vocab=1000), 4, 64, 8),
}
DEFAULT_WORKLOAD = "llama3-8b-shaped b32 p2048 d256"
FULL_SHAPE = dict(n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, d_ff=14336, vocab=128256)
# DRAM bytes one launch of gemm_tc_kernel with the SwiGLU epilogue at M=32, N=28672, K=4096 (bf16) moved under
# ncu (dram__bytes_read.sum + dram__bytes_write.sum; the capture summarised in profiles/ncu_gemm_m32_gateup.md)
NCU_TRAFFIC_GATEUP_M32 = 238.9e6


def host_threads():
    """Cores this process may use (its affinity mask, not the machine's core count)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def shape_of(workload):
    cfg_kw, batch, prompt, new = WORKLOADS[workload]
    full = dict(FULL_SHAPE)
    if cfg_kw:
        full.update(cfg_kw)
    return full, batch, prompt, new


def line_config(workload, replicas, parallelism):
    """``config`` of the JSON line: the workload and nothing measured, identical in both arms."""
    _, batch, prompt, new = shape_of(workload)
    return {"workload": workload, "global_batch": batch * replicas, "prompt_len": prompt, "new_tokens": new,
            "parallelism": parallelism}


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
# the reference's CPU path: stock PyTorch eager generation (infer.py with the kernels off)
# ---------------------------------------------------------------------------------------------
class CpuReference:
    """The workload's model on the host in fp32, at its full depth and width, generating on a
    bounded sample of the workload: batch 4, a 64-token prompt, 8 new tokens - the workload's own
    ratio of prompt to generated tokens (8 : 1), so that prefill and decode weigh as they do in
    it.  Every timed step is a real ``model.generate`` (infer.py:137-148 there); nothing is
    extrapolated.  The 8 G weights are N(0, 0.02) values tiled from one 16 M-element block:
    drawing each of them from the serial host generator would take minutes and the arithmetic
    does not depend on the values."""
    SAMPLE = (4, 64, 8)

    def __init__(self, workload):
        import torch
        from transformers import LlamaConfig, LlamaForCausalLM
        full, batch, prompt, new = shape_of(workload)
        self.threads = host_threads()
        torch.set_num_threads(self.threads)            # a launcher may have exported OMP_NUM_THREADS=1
        self.batch, self.prompt, self.new = min(batch, self.SAMPLE[0]), min(prompt, self.SAMPLE[1]), min(new, self.SAMPLE[2])
        hf = LlamaConfig(hidden_size=full["d_model"], intermediate_size=full["d_ff"], num_hidden_layers=full["n_layers"],
                         num_attention_heads=full["n_heads"], num_key_value_heads=full["n_kv_heads"], head_dim=full["head_dim"],
                         vocab_size=full["vocab"], rms_norm_eps=1e-5, rope_theta=5e5, max_position_embeddings=8192,
                         tie_word_embeddings=False)
        t0 = time.perf_counter()
        with torch.device("meta"):
            model = LlamaForCausalLM(hf)
        model = model.to_empty(device="cpu")
        block = torch.randn(1 << 24, generator=torch.Generator().manual_seed(0)) * 0.02
        with torch.no_grad():
            for name, p in model.named_parameters():
                if p.dim() == 1:
                    p.fill_(1.0)                       # norm weights
                    continue
                flat = p.view(-1)
                for lo in range(0, flat.numel(), block.numel()):
                    n = min(block.numel(), flat.numel() - lo)
                    flat[lo:lo + n].copy_(block[:n])
            for name, b in model.named_buffers():      # rotary inverse frequencies were left uninitialised by to_empty
                if "inv_freq" in name:
                    d = full["head_dim"]
                    b.copy_(1.0 / (5e5 ** (torch.arange(0, d, 2, dtype=torch.float32) / d)))
        self.model = model.eval()
        self.build_s = time.perf_counter() - t0
        self.ids = torch.randint(0, full["vocab"], (self.batch, self.prompt), generator=torch.Generator().manual_seed(1))
        self.layers = full["n_layers"]
        self.workload = workload

    def step(self):
        """Seconds of one greedy generation of the sample."""
        import torch
        t0 = time.perf_counter()
        with torch.no_grad():
            self.model.generate(self.ids, max_new_tokens=self.new, min_new_tokens=self.new, do_sample=False, pad_token_id=0)
        return time.perf_counter() - t0

    def tokens(self):
        return self.batch * self.new

    def describe(self, steps, sec):
        return (f"torch eager fp32 on {self.threads} host threads, HF LlamaForCausalLM at the workload's full shape "
                f"({self.layers} layers, weights built in {self.build_s:.0f} s), sample per step: batch {self.batch}, prompt "
                f"{self.prompt}, {self.new} new tokens (the workload's 8 : 1 prompt-to-new ratio); {steps} timed steps, "
                f"{sec:.2f} s per step, every step timed, nothing extrapolated")


def gpt2_small():
    """The reference's own CPU-runnable case: GPT-2-small shape, N(0, 0.02) weights from seed 0, fp32."""
    import torch
    from transformers import GPT2Config, GPT2LMHeadModel
    torch.manual_seed(0)
    cfg = GPT2Config(n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257, n_positions=1024,
                     initializer_range=0.02, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    model = GPT2LMHeadModel(cfg).eval()
    ids = torch.randint(0, 50257, (1, 128), generator=torch.Generator().manual_seed(0))
    return model, ids


def time_generate(model, ids, new, ctx_factory, sync, repeats=3):
    """infer.py's timed region (there :135-148): one warm-up, then the median of `repeats` generations."""
    import torch
    times = []
    for i in range(repeats + 1):
        sync()
        t0 = time.perf_counter()
        with torch.no_grad(), ctx_factory():
            out = model.generate(ids, max_new_tokens=new, min_new_tokens=new, do_sample=False, pad_token_id=0)
        sync()
        if i:
            times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2], out


def configs0_cpu():
    """GPT-2-small shape, batch 1, prompt 128, 64 greedy tokens, fp32 eager on the host cores."""
    import contextlib
    import torch
    threads = host_threads()
    torch.set_num_threads(threads)
    model, ids = gpt2_small()
    sec, _ = time_generate(model, ids, 64, contextlib.nullcontext, lambda: None)
    return {"workload": "gpt2-small-shaped fp32 b1 p128 d64", "cpu_eager_tok_s": 64 / sec, "cpu_s_per_generation": sec, "cores": threads,
            "timing": "one warm-up, median of 3 generations, wall clock around model.generate"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ref = CpuReference(args.workload)
    for _ in range(args.warmup):
        ref.step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ref.step()
    total = time.perf_counter() - t0
    v = ref.tokens() * args.steps / total
    replicas = max(1, args.gpus)
    line = {"impl": "reference", "metric": "decode+prefill tok/s", "value": v, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": line_config(args.workload, replicas, f"dp{replicas}"),
            "cpu_baseline": {"value": v, "unit": "tok/s", "cores": ref.threads, "kind": "port",
                             "sample": ref.describe(args.steps, total / args.steps)},
            "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    del ref
    gc.collect()
    try:
        line["configs0"] = configs0_cpu()
    except Exception as e:                # noqa: BLE001 - a secondary figure must not lose the line
        line["configs0"] = {"error": f"{type(e).__name__}: {e}"[:200]}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# this library: the plugin path (what a drop-in user runs)
# ---------------------------------------------------------------------------------------------
def hf_llama_on_gpu(full, dev, max_pos):
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM
    hf = LlamaConfig(hidden_size=full["d_model"], intermediate_size=full["d_ff"], num_hidden_layers=full["n_layers"],
                     num_attention_heads=full["n_heads"], num_key_value_heads=full["n_kv_heads"], head_dim=full["head_dim"],
                     vocab_size=full["vocab"], rms_norm_eps=1e-5, rope_theta=5e5, max_position_embeddings=max_pos,
                     tie_word_embeddings=False, initializer_range=0.02)
    torch.manual_seed(0)
    saved = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = LlamaForCausalLM(hf)
    finally:
        torch.set_default_dtype(saved)
    return model.eval()


class DispatchCounter:
    """Counts, per aten overload, the calls the op table served and the calls it handed back."""

    def __init__(self):
        import kuipy
        from kuipy import registry
        self.kuipy, self.real = kuipy, registry.try_dispatch
        self.hit, self.miss = {}, {}

    def __enter__(self):
        def counted(func, args, kwargs):
            out = self.real(func, args, kwargs)
            d = self.miss if out is None else self.hit
            d[str(func)] = d.get(str(func), 0) + 1
            return out
        self.kuipy._jit_dispatch = counted
        return self

    def __exit__(self, *exc):
        self.kuipy._jit_dispatch = self.real


def plugin_arms(workload, ids_host, dev, sizes):
    """The same generation by a HuggingFace Llama of the workload's shape, (a) eagerly under
    ``kuipy.KuiperMode()`` and (b) with its forward compiled by ``kuipy.inductor.backend``.  Host
    buffers: pinned ids in, generated ids back, inside the timed region.  Returns the ``plugin``
    object of the JSON line; a failing arm reports its error text instead of a number."""
    import torch
    import kuipy
    from kuipy import _ffi, inductor
    full, batch, prompt, new = shape_of(workload)
    res = {"model": "transformers LlamaForCausalLM, random init N(0, 0.02), bf16, DynamicCache (its per-token cat included)"}
    model = hf_llama_on_gpu(full, dev, prompt + new + 8)
    sync = lambda: torch.cuda.synchronize(dev)

    def generate(ids, n_new, ctx):
        with torch.no_grad(), ctx:
            out = model.generate(ids.to(dev, non_blocking=True), max_new_tokens=n_new, min_new_tokens=n_new, do_sample=False,
                                 pad_token_id=0)
            return out[:, ids.shape[1]:].to("cpu")

    def timed(ids, n_new, ctx_factory):
        sync()
        t0 = time.perf_counter()
        generate(ids, 1, ctx_factory())
        sync()
        t1 = time.perf_counter()
        generate(ids, n_new, ctx_factory())
        sync()
        t2 = time.perf_counter()
        total, prefill = t2 - t1, t1 - t0                              # infer_minimal.py:68-76: prefill = time to the first token
        return {"tok_s": ids.shape[0] * n_new / total, "s_per_generation": total, "prefill_s": prefill,
                "decode_ms_per_token": (total - prefill) / max(1, n_new - 1) * 1e3,
                "batch": ids.shape[0], "prompt_len": ids.shape[1], "new_tokens": n_new}

    # (a) the dispatch mode at the full workload
    try:
        with DispatchCounter() as cnt:
            generate(ids_host, 3, kuipy.KuiperMode())                    # warm-up, with the op census
        n0 = _ffi.launch_count()
        r = timed(ids_host, new, kuipy.KuiperMode)
        r["kuiops_launches"] = _ffi.launch_count() - n0
        r["census_of"] = "one prefill + 2 decode forwards"
        r["offloaded_calls"] = sum(cnt.hit.values())
        r["offloaded_ops"] = dict(sorted(cnt.hit.items(), key=lambda kv: -kv[1]))
        r["fall_through_ops"] = dict(sorted(cnt.miss.items(), key=lambda kv: -kv[1]))
        res["kuiper_mode"] = r
    except Exception as e:                # noqa: BLE001
        res["kuiper_mode"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    # stock PyTorch eager on the same GPU and model, for scale (cuBLAS / flash-attention library kernels)
    try:
        import contextlib
        generate(ids_host, 3, contextlib.nullcontext())
        res["torch_eager_gpu"] = timed(ids_host, new, contextlib.nullcontext)
    except Exception as e:                # noqa: BLE001
        res["torch_eager_gpu"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    # (b) the graph front end.  Under torch.compile HuggingFace materialises its causal mask, so attention
    # arrives as the efficient overload with an additive bias, which the tcgen05 flash kernel does not take
    # (the SIMT kernel does): the arm runs on a bounded sample of the workload, stated in the result.
    try:
        import torch._dynamo
        sb, sp, sn = sizes
        ids_small = ids_host[:sb, :sp].contiguous().pin_memory()
        torch._dynamo.reset()
        eager_forward = model.forward
        model.forward = torch.compile(eager_forward, backend=inductor.backend)
        before = {k: list(v) for k, v in inductor.call_stats.items()}
        generate(ids_small, 3, torch.no_grad())                          # compiles the prefill and the decode graph
        n0 = _ffi.launch_count()
        r = timed(ids_small, sn, torch.no_grad)
        r["kuiops_launches"] = _ffi.launch_count() - n0
        r["served_by_kuiops"] = {k: v[0] - before.get(k, [0, 0])[0] for k, v in inductor.call_stats.items() if v[0] - before.get(k, [0, 0])[0]}
        r["handed_back"] = {k: v[1] - before.get(k, [0, 0])[1] for k, v in inductor.call_stats.items() if v[1] - before.get(k, [0, 0])[1]}
        r["note"] = "bounded sample: attention arrives with an explicit mask under torch.compile and runs on the SIMT kernel"
        res["inductor_backend"] = r
        model.forward = eager_forward
    except Exception as e:                # noqa: BLE001
        res["inductor_backend"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    if _ffi.tc_error() != 0:
        res["tc_error"] = "a tensor-core pipeline wait timed out"
    del model
    gc.collect()
    torch.cuda.empty_cache()
    return res


def configs0_pair(dev):
    """configs0 on both sides: host cores with the kernels off, and this GPU under KuiperMode."""
    import torch
    import kuipy
    from kuipy import _ffi
    out = configs0_cpu()
    model, ids = gpt2_small()
    model = model.to(dev)
    ids = ids.to(dev)
    n0 = _ffi.launch_count()
    sec, _ = time_generate(model, ids, 64, kuipy.KuiperMode, lambda: torch.cuda.synchronize(dev))
    out.update({"kuiper_mode_gpu_tok_s": 64 / sec, "gpu_s_per_generation": sec, "kuiops_launches": _ffi.launch_count() - n0})
    return out


# ---------------------------------------------------------------------------------------------
# this library: the decoder harness (C ABI), data parallel and tensor parallel
# ---------------------------------------------------------------------------------------------
def time_decoder(dec, cfg, batch, prompt, new, ids_dev, ids_host, dev, steps, warmup, use_graph, barrier, sampler=None):
    """W warm-up generations, then K timed ones (device-resident ids), then K more through host
    buffers.  Returns the timings in ms and the number of kuiops kernels launched."""
    import torch
    from kuipy import _ffi
    ev = lambda: torch.cuda.Event(enable_timing=True)
    out_host = torch.empty((batch, new), dtype=torch.int64).pin_memory()
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
        tok = dec.next_token(dec.prefill(ids, local_logits=True))
        gen_buf[:, 0].copy_(tok)
        if marks is not None:
            marks[1].record()
        if use_graph:
            dec.decode_graph(tok, new - 1, out=gen_buf[:, 1:])
            replays[0] += new - 1
        else:
            for t in range(1, new):
                tok = dec.next_token(dec.decode_step(tok, local_logits=True))
                gen_buf[:, t].copy_(tok)
        if marks is not None:
            marks[2].record()
        return gen_buf

    for _ in range(warmup):
        one_step(ids_dev)
    barrier()
    if sampler is not None:
        sampler.start()
    marks = [[ev(), ev(), ev()] for _ in range(steps)]
    n0 = _ffi.launch_count()
    replays[0] = 0
    barrier()
    t_start, t_end = ev(), ev()
    t_start.record()
    for s in range(steps):
        one_step(ids_dev, marks[s])
    t_end.record()
    barrier()
    launches = _ffi.launch_count() - n0 + (replays[0] * dec.graph_launches if use_graph else 0)
    clocks = sampler.stop() if sampler is not None else None
    total_ms = t_start.elapsed_time(t_end)
    prefill_ms = sum(m[0].elapsed_time(m[1]) for m in marks) / steps
    decode_ms = sum(m[1].elapsed_time(m[2]) for m in marks) / steps
    # end to end through the public call with host buffers: pinned ids in, generated ids out
    barrier()
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(steps):
        ids_in = ids_host.to(dev, non_blocking=True)
        out_host.copy_(one_step(ids_in), non_blocking=True)
    e1.record()
    barrier()
    return dict(total_ms=total_ms, prefill_ms=prefill_ms, decode_ms=decode_ms, e2e_ms=e0.elapsed_time(e1), launches=launches,
                clocks=clocks, out_bytes=out_host.numel() * 8)


def gateup_roofline(dec, cfg, batch, dev, tp):
    """Roofline of the dominant decode kernel: the gate|up weight-streaming GEMM with its fused SwiGLU
    epilogue, exactly the launch the decode step makes, timed live over the layers' distinct weights
    (7.5 GB at the 8B shape, far beyond L2): the launches are replayed from a CUDA graph, as in the
    decode step, with events on the replaying stream."""
    import torch
    from kuipy import _ffi
    ev = lambda: torch.cuda.Event(enable_timing=True)
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
    traffic = NCU_TRAFFIC_GATEUP_M32 if (n_out, k_in, batch, tp) == (28672, 4096, 32, 1) else None
    return {"kernel": "gemm_tc_kernel (gate|up projection + SwiGLU epilogue of one decode step)", "bound": "hbm",
            "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
            "peak_kind": peak_kind, "nominal_peak": 8000.0, "frac_nominal": achieved / 8000.0,
            "traffic": traffic, "traffic_source": "ncu capture of this launch shape (profiles/ncu_gemm_m32_gateup.md)" if traffic else None,
            "us_per_launch": gemm_ms * 1e3, "algorithmic_bytes_per_launch": alg_bytes}


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

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(vals):
        t = torch.tensor(vals, device=dev, dtype=torch.float64)
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    cfg_kw, batch, prompt, new = WORKLOADS[args.workload]
    cfg = DecoderConfig(**cfg_kw) if cfg_kw else DecoderConfig.llama3_8b()
    use_graph = not args.no_graph
    only_tp = args.parallel == "tp" and world > 1
    line = None

    # ---- batch data parallel: one full replica and its own batch per rank, no collective --------------
    if not only_tp:
        dec = Decoder(cfg, device=dev, seed=0)
        dec.alloc_cache(batch, prompt + new)
        g = torch.Generator().manual_seed(1000 + rank)
        ids_host = torch.randint(0, cfg.vocab, (batch, prompt), generator=g).pin_memory()
        ids_dev = ids_host.to(dev)
        sampler = ClockSampler(local) if rank == 0 else None
        t = time_decoder(dec, cfg, batch, prompt, new, ids_dev, ids_host, dev, args.steps, args.warmup, use_graph, barrier, sampler)
        word = _ffi.tc_error()
        if word != 0:
            raise SystemExit(f"a tensor-core pipeline wait timed out during the bench (error word {word}); numbers discarded")
        roofline = gateup_roofline(dec, cfg, batch, dev, 1)
        total_ms, e2e_ms, prefill_ms, decode_ms = max_over_ranks([t["total_ms"], t["e2e_ms"], t["prefill_ms"], t["decode_ms"]])
        gen_tokens = batch * new * world * args.steps
        if rank == 0:
            line = {
                "metric": "decode+prefill tok/s", "value": gen_tokens / (total_ms * 1e-3), "unit": "tok/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": line_config(args.workload, world, f"dp{world}"),
                "detail": {"decode_cuda_graph": use_graph,
                           "prefill_tok_s": batch * prompt * world / (prefill_ms * 1e-3),
                           "decode_tok_s": batch * (new - 1) * world / (decode_ms * 1e-3),
                           "prefill_ms": prefill_ms, "decode_ms_per_token": decode_ms / (new - 1),
                           "l2": "weights streamed per step (15 GB at the 8B shape) exceed the 126 MB L2; no flush"},
                "e2e": {"value": gen_tokens / (e2e_ms * 1e-3), "unit": "tok/s", "through": "C ABI (kuillm_b200.decoder), pinned host ids in, generated ids out",
                        "h2d_bytes_per_step": ids_host.numel() * 8, "d2h_bytes_per_step": t["out_bytes"]},
                "gpu_launches": t["launches"],
                "clocks": t["clocks"],
                "roofline": roofline,
            }
        dec._graph = None
        del dec, ids_dev
        gc.collect()
        torch.cuda.empty_cache()

    # ---- tensor parallel over all ranks: one global batch, two sums over ranks per layer ---------------
    if world > 1:
        tp_res = {}
        try:
            import torch.distributed as dist
            tp_steps, tp_warm = max(1, min(args.steps, args.tp_steps)), max(1, min(args.warmup, 2))
            dec = Decoder(cfg, device=dev, seed=0, tp_rank=rank, tp_size=world)
            dec.alloc_cache(batch, prompt + new)
            fused = args.allreduce == "fused"
            fused_note = ""
            if fused:
                # decode steps only (batch rows); the prefill keeps NCCL.  The fused form needs every rank's receive
                # area mapped into every process; where that cannot be had the step keeps NCCL, and says so
                try:
                    dec.enable_fused_allreduce(batch)
                    ok = torch.ones(1, device=dev)
                except Exception as e:            # noqa: BLE001 - whatever the mapping raised is reported, not hidden
                    fused_note = f"{type(e).__name__}: {e}"[:160]
                    ok = torch.zeros(1, device=dev)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                if ok.item() == 0:
                    dec.exchange, fused = None, False
            g = torch.Generator().manual_seed(1000)
            ids_host = torch.randint(0, cfg.vocab, (batch, prompt), generator=g).pin_memory()
            ids_dev = ids_host.to(dev)
            if fused:
                # one trial decode step before anything is timed: an exchange that does not work on this group
                # shows here within about a minute (its waits are bounded, 1 s each for the trial) instead of
                # stretching every step of the measurement; the step then keeps NCCL, and the line says so
                old_wait = _ffi.set_peer_wait_ns(1_000_000_000)
                dec.length = 0
                tok = dec.next_token(dec.prefill(ids_dev[:, :8].contiguous(), local_logits=True))
                dec.next_token(dec.decode_step(tok, local_logits=True))
                torch.cuda.synchronize()
                bad = torch.tensor([1.0 if _ffi.tc_error() != 0 else 0.0], device=dev)
                dist.all_reduce(bad, op=dist.ReduceOp.MAX)
                _ffi.set_peer_wait_ns(old_wait)
                dec.length = 0
                if bad.item() != 0:
                    dec.exchange, fused = None, False
                    fused_note = "a bounded wait of the fused exchange ran out in the trial step"
            t = time_decoder(dec, cfg, batch, prompt, new, ids_dev, ids_host, dev, tp_steps, tp_warm, use_graph, barrier)
            total_ms, e2e_ms, prefill_ms, decode_ms = max_over_ranks([t["total_ms"], t["e2e_ms"], t["prefill_ms"], t["decode_ms"]])
            tp_res = {"parallelism": f"tp{world}", "scaling": "strong", "global_batch": batch, "steps": tp_steps, "warmup": tp_warm,
                      "tok_s": batch * new * tp_steps / (total_ms * 1e-3), "e2e_tok_s": batch * new * tp_steps / (e2e_ms * 1e-3),
                      "ms_per_step": total_ms / tp_steps, "prefill_ms": prefill_ms, "decode_ms_per_token": decode_ms / (new - 1),
                      "decode_allreduce": "fused into the GEMM epilogue and the next norm (peer stores)" if fused else "nccl",
                      "prefill_allreduce": "nccl", "gpu_launches": t["launches"]}
            if fused_note:
                tp_res["fused_unavailable"] = fused_note
            if _ffi.tc_error() != 0:
                tp_res["error"] = "a bounded device wait ran out; numbers unreliable"
            dec._graph = None
            del dec
        except Exception as e:                    # noqa: BLE001
            tp_res = {"error": f"{type(e).__name__}: {e}"[:300]}
        if rank == 0:
            if line is None:                       # --parallel tp: the tensor-parallel form is the line itself
                line = {"metric": "decode+prefill tok/s", "value": tp_res.get("tok_s"), "unit": "tok/s", "n_gpus": world,
                        "steps": tp_res.get("steps"), "warmup": tp_res.get("warmup"), "ms_per_step": tp_res.get("ms_per_step"),
                        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                        "config": line_config(args.workload, 1, f"tp{world}"), "detail": tp_res,
                        "e2e": {"value": tp_res.get("e2e_tok_s"), "unit": "tok/s", "h2d_bytes_per_step": batch * prompt * 8,
                                "d2h_bytes_per_step": batch * new * 8},
                        "gpu_launches": tp_res.get("gpu_launches")}
            else:
                line["tp"] = tp_res
        gc.collect()
        torch.cuda.empty_cache()

    # ---- rank 0 of a single-GPU run: the plugin path, configs0, the operator table, the host baseline ----
    if rank == 0 and world == 1 and line is not None:
        if not args.no_plugin:
            try:
                line["plugin"] = plugin_arms(args.workload, ids_host, dev, (4, 512, 32))
            except Exception as e:                # noqa: BLE001
                line["plugin"] = {"error": f"{type(e).__name__}: {e}"[:300]}
            try:
                line["configs0"] = configs0_pair(dev)
            except Exception as e:                # noqa: BLE001
                line["configs0"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        if not args.no_op_table:
            try:
                from kuillm_b200 import opbench
                time.sleep(3.0)                   # the generation above ran at the power cap
                rows, kind = opbench.baseline_sweep(iters=20)
                line["op_table"] = {"peak_kind": kind, "columns": ["op", "shape", "us", "bound", "frac of measured peak", "frac of nominal (8 TB/s, 2.25 PFLOP/s)"],
                                    "rows": [[r["op"], r["shape"], r["us"], r["bound"], r["frac"], r["frac_nominal"]] for r in rows]}
            except Exception as e:                # noqa: BLE001
                line["op_table"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        if not args.no_cpu_baseline:
            torch.cuda.empty_cache()
            ref = CpuReference(args.workload)
            ref.step()
            n = 3
            t0 = time.perf_counter()
            for _ in range(n):
                ref.step()
            sec = (time.perf_counter() - t0) / n
            line["cpu_baseline"] = {"value": ref.tokens() / sec, "unit": "tok/s", "cores": ref.threads, "kind": "port",
                                    "sample": ref.describe(n, sec)}
            del ref
    if rank == 0 and line is not None:
        print(json.dumps(line))
    if world > 1:
        # a captured graph may hold NCCL work: drain the device before the ranks part, then leave without
        # tearing the communicator down (teardown after graph capture can block)
        import torch.distributed as dist
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
    ap.add_argument("--parallel", default="dp", choices=["dp", "tp"],
                    help="with N > 1: 'dp' runs the data-parallel arm and then the tensor-parallel one; 'tp' only the latter")
    ap.add_argument("--tp-steps", type=int, default=5, help="timed steps of the tensor-parallel arm (at most --steps)")
    ap.add_argument("--allreduce", default="fused", choices=["fused", "nccl"],
                    help="tensor parallel only: how the decode step sums the row-split projections")
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=list(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-plugin", action="store_true", help="skip the HuggingFace-under-KuiperMode / compiled arms and configs0")
    ap.add_argument("--no-op-table", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every decode kernel from the host instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
