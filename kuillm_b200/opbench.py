"""Per-operator roofline table at the benchmark configurations.

    python -m kuillm_b200.opbench [--only stream,index,decode,sdpa,gemm] [--iters 20] [--out file.jsonl]

Each line: op, shape, microseconds per launch (CUDA events on the launching stream, after
warm-up), the algorithmic bytes or flops of one launch, the achieved rate and its fraction of
this pool's measured peak (MEASURED_PEAKS.json next to the repository root, else the fallback
6650 GB/s / 1590 TFLOP/s), and of the nominal 8 TB/s / 2.25 PFLOP/s.  Memory-bound ops rotate over enough distinct input buffers that the
working set exceeds the 126 MB L2.
"""
import argparse
import json
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
for _p in (ROOT, ROOT / "kuillm_b200"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))
from kuipy import _ffi  # noqa: E402

L2_BYTES = 126 << 20


def peaks():
    try:
        d = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    except (OSError, ValueError, KeyError):
        return 6650.0, 1590.0, "fallback"


_side = None
EAGER = False        # --eager: plain launches timed with events (what a profiler capture needs)
MATCH = ""           # --match: only time cases whose "op shape" contains this text


def wanted(op, shape):
    return MATCH in f"{op} {shape}"


def time_us(fn, n_variants, iters):
    """Average device time of fn(i % n_variants) over `iters` launches.  The launches are captured
    in a CUDA graph and the replay is timed, so host-side launch cost (tens of microseconds per call
    through Python) does not hide kernels that run for a few microseconds."""
    global _side
    if EAGER:
        for i in range(2):
            fn(i % n_variants)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(i % n_variants)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / iters
    if _side is None:
        _side = torch.cuda.Stream()
    _side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(_side):
        for i in range(min(3, n_variants) + 2):
            fn(i % n_variants)
        _side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=_side):
            for i in range(iters):
                fn(i % n_variants)
        graph.replay()
        _side.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(_side)
        graph.replay()
        e1.record(_side)
        _side.synchronize()
    torch.cuda.current_stream().wait_stream(_side)
    del graph
    return e0.elapsed_time(e1) * 1e3 / iters


def variants_for(bytes_per_input):
    return max(2, min(64, -(-2 * L2_BYTES // max(1, bytes_per_input))))


class Table:
    def __init__(self, out, quiet=False):
        self.hbm, self.tf, self.kind = peaks()
        self.rows, self.out, self.quiet = [], out, quiet

    def add(self, op, shape, us, bytes_=None, flops=None, bound="hbm", note=""):
        if callable(us):
            if not wanted(op, shape):
                return
            us = us()
        row = {"op": op, "shape": shape, "us": round(us, 2), "bound": bound, "peak_kind": self.kind}
        if bytes_ is not None:
            row["alg_bytes"] = int(bytes_)
            row["GBps"] = round(bytes_ / us / 1e3, 1)
        if flops is not None:
            row["alg_flops"] = int(flops)
            row["TFLOPs"] = round(flops / us / 1e6, 1)
        row["frac"] = round((row["GBps"] / self.hbm) if bound == "hbm" else (row["TFLOPs"] / self.tf), 3)
        # the same against the data-sheet figures (8 TB/s HBM3e, 2.25 PFLOP/s dense bf16)
        row["frac_nominal"] = round((row["GBps"] / 8000.0) if bound == "hbm" else (row["TFLOPs"] / 2250.0), 3)
        if note:
            row["note"] = note
        self.rows.append(row)
        if not self.quiet:
            print(json.dumps(row), flush=True)
        if self.out:
            with open(self.out, "a") as f:
                f.write(json.dumps(row) + "\n")


def bench_stream(T, iters):
    dev = "cuda"
    m, n = 64, 128256
    if any(wanted(o, f"{m}x{n}") for o in ("softmax_f32", "topk_f32_k50", "argmax_f32", "cumsum_f32", "sort_f32", "multinomial_f32", "sample_topk50_topp_f32")):
        nv = variants_for(m * n * 4)
        xs = [torch.randn(m, n, device=dev) * 3 for _ in range(nv)]
        y = torch.empty_like(xs[0])
        T.add("softmax_f32", f"{m}x{n}", (lambda: time_us(lambda i: _ffi.softmax(xs[i], out=y), nv, iters)), bytes_=2 * m * n * 4)
        if wanted("topk_f32_k50", f"{m}x{n}"):
            ps = [_ffi.softmax(x) for x in xs]
            T.add("topk_f32_k50", f"{m}x{n}", (lambda: time_us(lambda i: _ffi.topk(ps[i], 50), nv, iters)), bytes_=m * n * 4 + m * 50 * 12)
            del ps
        T.add("argmax_f32", f"{m}x{n}", (lambda: time_us(lambda i: _ffi.argmax_lastdim(xs[i]), nv, iters)), bytes_=m * n * 4)
        if wanted("multinomial_f32", f"{m}x{n}"):
            pm = [_ffi.softmax(x) for x in xs]
            T.add("multinomial_f32", f"{m}x{n}", (lambda: time_us(lambda i: _ffi.multinomial(pm[i], 1, seed=1, offset=4 * i), nv, iters)), bytes_=m * n * 4,
                  note="one draw per row; one CTA per row")
            del pm
        if wanted("sample_topk50_topp_f32", f"{m}x{n}"):
            ids = torch.empty(m, dtype=torch.int64, device=dev)
            T.add("sample_topk50_topp_f32", f"{m}x{n}",
                  (lambda: time_us(lambda i: _ffi.sample_topk_topp(xs[i], 0.7, 50, 0.8, seed=1, offset=4 * i, out=ids), nv, iters)), bytes_=m * n * 4,
                  note="temperature + top-k + top-p + draw: two launches, the logits read once")
        T.add("sort_f32", f"{m}x{n}", (lambda: time_us(lambda i: _ffi.sort_lastdim(xs[i]), nv, max(2, iters // 4))), bytes_=m * n * 16,
              note="values + int64 permutation; a cluster of 4 CTAs per row")
        T.add("cumsum_f32", f"{m}x{n}", (lambda: time_us(lambda i: _ffi.cumsum_lastdim(xs[i], out=y), nv, iters)), bytes_=2 * m * n * 4)
        del xs
    if wanted("reduce_max_f32", "8208384"):
        nv = variants_for(m * n * 4)
        fl = [torch.randn(m * n, device=dev) for _ in range(nv)]
        T.add("reduce_max_f32", f"{m * n}", (lambda: time_us(lambda i: _ffi.reduce("max", fl[i]), nv, iters)), bytes_=m * n * 4)
        T.add("mean_f32_lastdim", f"{m}x{n}", (lambda: time_us(lambda i: _ffi.mean_lastdim(fl[i].view(m, n)), nv, iters)), bytes_=m * n * 4)
        del fl
    if wanted("argmax_bf16", "32x128256"):
        nv = variants_for(32 * n * 2)
        lb = [torch.randn(32, n, device=dev).bfloat16() for _ in range(nv)]
        T.add("argmax_bf16", f"32x{n}", (lambda: time_us(lambda i: _ffi.argmax_lastdim(lb[i]), nv, iters)), bytes_=32 * n * 2)
        del lb
    if wanted("softmax_f32", "4096x32768"):
        big = [torch.randn(4096, 32768, device=dev) for _ in range(2)]
        yb2 = torch.empty_like(big[0])
        T.add("softmax_f32", "4096x32768", (lambda: time_us(lambda i: _ffi.softmax(big[i % 2], out=yb2), 2, iters)), bytes_=2 * 4096 * 32768 * 4)
        del big, yb2
    rows, d = 32 * 2048, 4096
    if any(wanted(o, f"{rows}x{d}") or wanted(o, f"{rows * d}") for o in ("mean_f32_lastdim", "reduce_max_f32")):
        nv = variants_for(rows * d * 4)
        hs = [torch.randn(rows, d, device=dev) for _ in range(nv)]
        T.add("mean_f32_lastdim", f"{rows}x{d}", (lambda: time_us(lambda i: _ffi.mean_lastdim(hs[i]), nv, iters)), bytes_=rows * d * 4)
        T.add("reduce_max_f32", f"{rows * d}", (lambda: time_us(lambda i: _ffi.reduce("max", hs[i]), nv, iters)), bytes_=rows * d * 4)
        del hs
    if any(wanted(o, f"{rows}x{d}") or wanted(o, f"{rows * d}") for o in ("rmsnorm_bf16", "map_silu_bf16", "map2_add_bf16")):
        hb = [torch.randn(rows, d, device=dev).bfloat16() for _ in range(2)]
        w = torch.ones(d, device=dev, dtype=torch.bfloat16)
        yb = torch.empty_like(hb[0])
        T.add("rmsnorm_bf16", f"{rows}x{d}", (lambda: time_us(lambda i: _ffi.rmsnorm(hb[i % 2], w, 1e-5, out=yb), 2, iters)),
              bytes_=2 * rows * d * 2)
        T.add("map_silu_bf16", f"{rows * d}", (lambda: time_us(lambda i: _ffi.map1("silu", hb[i % 2], out=yb), 2, iters)),
              bytes_=2 * rows * d * 2)
        T.add("map2_add_bf16", f"{rows * d}", (lambda: time_us(lambda i: _ffi.map2("add", hb[i % 2], hb[(i + 1) % 2], out=yb), 2, iters)),
              bytes_=3 * rows * d * 2)


def bench_index(T, iters):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    for (r, c) in ((64, 2048), (8192, 16384)):
        nb = r * c * 8
        nv = variants_for(nb)
        ids = [torch.randint(0, 128256, (r, c), device=dev, generator=g) for _ in range(nv)]
        idx = torch.randint(0, c, (r, c), device=dev, generator=g)
        perm = torch.argsort(torch.rand(r, c, device=dev, generator=g), dim=1)
        T.add("gather_i64_dim1", f"{r}x{c}", (lambda: time_us(lambda i: _ffi.gather(ids[i], 1, idx), nv, iters)), bytes_=3 * nb,
              note="payload in + index in + out")
        T.add("scatter_i64_dim1", f"{r}x{c}", (lambda: time_us(lambda i: _ffi.scatter(ids[i], 1, perm, ids[(i + 1) % nv]), nv, iters)),
              bytes_=4 * nb, note="self in + src + index + out")
        pos = torch.randint(0, c, (c // 4,), device=dev, generator=g)
        T.add("index_i64_dim1", f"{r}x{c}[:, {c // 4}]", (lambda: time_us(lambda i: _ffi.index(ids[i], 1, [pos]), nv, iters)),
              bytes_=2 * r * (c // 4) * 8)
        stop = torch.randint(0, 128256, (1024,), device=dev, generator=g)
        T.add("isin_i64_vs_1024", f"{r}x{c}", (lambda: time_us(lambda i: _ffi.isin(ids[i], stop), nv, iters)), bytes_=nb + r * c)
        parts = [[t[:, k * (c // 8):(k + 1) * (c // 8)].contiguous() for k in range(8)] for t in ids[:max(2, nv // 2)]]
        T.add("cat_8_slices_dim1", f"8 x {r}x{c // 8}", (lambda: time_us(lambda i: _ffi.cat(parts[i % len(parts)], 1), len(parts), iters)),
              bytes_=2 * nb)
        del ids, parts


def bench_gemm(T, iters):
    dev = "cuda"
    if wanted("gemm_swiglu_bf16_tn", "M32 N28672 K4096"):
        N, K, M = 28672, 4096, 32
        nv = variants_for(N * K * 2)
        Ws = [(torch.randn(N, K, device=dev) / K ** 0.5).bfloat16() for _ in range(nv)]
        A = torch.randn(M, K, device=dev).bfloat16()
        T.add("gemm_swiglu_bf16_tn", f"M{M} N{N} K{K}", (lambda: time_us(lambda i: _ffi.gemm_swiglu(A, Ws[i]), nv, iters)),
              bytes_=2 * (N * K + M * K + M * N // 2), flops=2 * M * N * K, bound="hbm", note="gate|up projection with the SwiGLU epilogue")
        del Ws
    for (N, K) in ((4096, 4096), (6144, 4096), (14336, 4096), (28672, 4096), (4096, 14336), (128256, 4096)):
        if MATCH and not any(wanted(o, f"M{M} N{N} K{K}") for o in ("gemm_bf16_tn", "addmm_bias_bf16_tn") for M in (1, 8, 16, 32, 128, 4096)):
            continue
        nv = variants_for(N * K * 2)
        Ws = [(torch.randn(N, K, device=dev) / K ** 0.5).bfloat16() for _ in range(min(nv, 6 if N > 100000 else nv))]
        bias = torch.zeros(N, device=dev, dtype=torch.bfloat16)
        for M in (1, 8, 16, 32, 128, 4096):
            if not wanted("gemm_bf16_tn", f"M{M} N{N} K{K}") and not wanted("addmm_bias_bf16_tn", f"M{M} N{N} K{K}"):
                continue
            A = torch.randn(M, K, device=dev).bfloat16()
            C = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            us = (lambda: time_us(lambda i: _ffi.gemm(A, Ws[i % len(Ws)], trans_b=True, out=C), len(Ws), iters))
            by, fl = 2 * (M * K + N * K + M * N), 2 * M * N * K
            if M >= 4096:
                T.add("gemm_bf16_tn", f"M{M} N{N} K{K}", us, bytes_=by, flops=fl, bound="tensor")
            else:
                T.add("gemm_bf16_tn", f"M{M} N{N} K{K}", us, bytes_=by, flops=fl, bound="hbm")
            if M in (16, 4096) and N == 4096 and K == 4096:
                us = (lambda: time_us(lambda i: _ffi.gemm(A, Ws[i % len(Ws)], trans_b=True, Cin=bias, out=C), len(Ws), iters))
                T.add("addmm_bias_bf16_tn", f"M{M} N{N} K{K}", us, bytes_=by, flops=fl, bound="tensor" if M >= 4096 else "hbm")
        del Ws
    if not MATCH or any(wanted(o, "") for o in ("mm_bf16_nn", "bmm_bf16", "mm_f32_simt")):
        # row-major B (MN-major tiles), the aten.mm operand form
        A = torch.randn(4096, 4096, device=dev).bfloat16()
        Bs = [(torch.randn(4096, 4096, device=dev) / 64).bfloat16() for _ in range(8)]
        T.add("mm_bf16_nn", "M4096 N4096 K4096", (lambda: time_us(lambda i: _ffi.mm(A, Bs[i % 8]), 8, iters)), flops=2 * 4096 ** 3,
              bytes_=3 * 2 * 4096 ** 2, bound="tensor")
        A3 = [torch.randn(32, 4096, 128, device=dev).bfloat16() for _ in range(4)]
        B3 = [(torch.randn(32, 128, 4096, device=dev) / 11.3).bfloat16() for _ in range(4)]
        T.add("bmm_bf16", "32 x 4096x128x4096", (lambda: time_us(lambda i: _ffi.bmm(A3[i % 4], B3[i % 4]), 4, iters)),
              bytes_=2 * 32 * (2 * 4096 * 128 + 4096 * 4096), flops=2 * 32 * 4096 * 128 * 4096, bound="hbm")
        A32 = torch.randn(4096, 4096, device=dev)
        B32 = torch.randn(4096, 4096, device=dev) / 64
        T.add("mm_f32_simt", "M4096 N4096 K4096", (lambda: time_us(lambda i: _ffi.mm(A32, B32), 1, max(3, iters // 4))), flops=2 * 4096 ** 3,
              bytes_=3 * 4 * 4096 ** 2, bound="tensor", note="SIMT fp32 path; fraction is against the bf16 tensor peak")

        del A, Bs, A3, B3, A32, B32
    # the prefill shapes of the whole-model benchmark: 32 x 2048 rows at once (last: tens of
    # milliseconds of dense tensor work heat the part and would depress whatever is timed next)
    for (N, K) in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)):
        M = 65536
        if not wanted("gemm_bf16_tn", f"M{M} N{N} K{K}"):
            continue
        A = torch.randn(M, K, device=dev).bfloat16()
        W = (torch.randn(N, K, device=dev) / K ** 0.5).bfloat16()
        C = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        T.add("gemm_bf16_tn", f"M{M} N{N} K{K}", (lambda: time_us(lambda i: _ffi.gemm(A, W, trans_b=True, out=C), 1, max(2, iters // 4))),
              bytes_=2 * (M * K + N * K + M * N), flops=2 * M * N * K, bound="tensor")
        del A, W, C


def _sdpa_decode_cases(T, iters, hkv):
    dev = "cuda"
    D = 128
    for S in (4096, 32768):
        B, H = 64, 32
        if not wanted("sdpa_decode_bf16", f"B{B} Hq{H} Hkv{hkv} Skv{S} D{D}"):
            continue
        kv_bytes = 2 * B * hkv * S * D * 2
        nv = variants_for(kv_bytes) if kv_bytes < (8 << 30) else 1
        nv = min(nv, 2)
        Q = torch.randn(B, H, 1, D, device=dev).bfloat16()
        Ks = [torch.randn(B, hkv, S, D, device=dev).bfloat16() for _ in range(nv)]
        Vs = [torch.randn(B, hkv, S, D, device=dev).bfloat16() for _ in range(nv)]
        O = torch.empty_like(Q)
        us = (lambda: time_us(lambda i: _ffi.sdpa(Q, Ks[i], Vs[i], is_causal=True, need_lse=False, out=O), nv, max(3, iters // 2)))
        T.add("sdpa_decode_bf16", f"B{B} Hq{H} Hkv{hkv} Skv{S} D{D}", us, bytes_=kv_bytes + 2 * B * H * D * 2 * 2,
              flops=4 * B * H * S * D, bound="hbm")
        del Ks, Vs



def bench_sdpa(T, iters):
    dev = "cuda"
    D = 128
    # decode (memory bound) first: seconds of dense tensor work in the prefill cases heat the
    # part and would depress whatever is timed right after them
    for hkv in (32, 8):
        _sdpa_decode_cases(T, iters, hkv)
    for hkv in (32, 8):
        for S in (1024, 4096, 16384):
            B, H = 8, 32
            if not wanted("sdpa_prefill_causal_bf16", f"B{B} Hq{H} Hkv{hkv} S{S} D{D}"):
                continue
            Q = torch.randn(B, H, S, D, device=dev).bfloat16()
            K = torch.randn(B, hkv, S, D, device=dev).bfloat16()
            V = torch.randn(B, hkv, S, D, device=dev).bfloat16()
            O = torch.empty_like(Q)
            it = max(2, iters // (4 if S >= 16384 else 1))
            us = (lambda: time_us(lambda i: _ffi.sdpa(Q, K, V, is_causal=True, need_lse=False, out=O), 1, it))
            T.add("sdpa_prefill_causal_bf16", f"B{B} Hq{H} Hkv{hkv} S{S} D{D}", us, flops=2 * B * H * S * S * D,
                  bytes_=2 * (2 * B * H * S * D + 2 * B * hkv * S * D), bound="tensor")
            del Q, K, V, O


def bench_decode_breakdown(T, iters):
    """Where one decode step of the Llama-3-8B shape (batch 32, context 2176) spends its time:
    the step's kernels are replayed group by group from CUDA graphs (same weights, caches and
    launch arguments as the real step), next to the whole captured step."""
    from kuillm_b200.decoder import Decoder, DecoderConfig
    cfg = DecoderConfig.llama3_8b()
    B, cap, ctx = 32, 2304, 2176
    dec = Decoder(cfg)
    dec.alloc_cache(B, cap)
    dev = dec.device
    hd, hq, hk, d = cfg.head_dim, dec.hq, dec.hk, cfg.d_model
    W = (hq + 2 * hk) * hd
    x = torch.randn(B, d, device=dev).bfloat16()
    resid = torch.randn(B, d, device=dev).bfloat16()
    qkv = torch.randn(B, W, device=dev).bfloat16()
    attn = torch.randn(B, hq * hd, device=dev).bfloat16()
    act = torch.randn(B, dec.ff, device=dev).bfloat16()
    pos = torch.full((B,), ctx - 1, device=dev, dtype=torch.int64)
    kvlen = torch.full((B,), ctx, device=dev, dtype=torch.int64)
    q4 = qkv.as_strided((B, hq, 1, hd), (W, hd, W, 1))
    o4 = attn.as_strided((B, hq, 1, hd), (hq * hd, hd, hq * hd, 1))
    tok = torch.zeros(B, dtype=torch.int64, device=dev)

    tiles = _ffi.ssq_tiles(d)
    ssq_a = torch.rand(tiles, B, device=dev) * 128 + 64
    ssq_b = torch.rand(tiles, B, device=dev) * 128 + 64

    def gemms():
        # the four projections of a layer as the step launches them: both RMSNorms are folded in
        for li, L in enumerate(dec.layers):
            _ffi.gemm_rope_qkv_rms(resid, L["wqkv"], hq, hk, hd, pos, cfg.rope_theta, ssq_a, cfg.eps, dec.k_cache[li], dec.v_cache[li],
                                   rows_per_seq=1, out=qkv)
            _ffi.gemm_residual_ssq(attn, L["wo"], resid, ssq_b)
            _ffi.gemm_swiglu_rms(resid, L["wgu"], ssq_b, cfg.eps)
            _ffi.gemm_residual_ssq(act, L["wd"], resid, ssq_a)       # (the running sum grows over the replays; timing does not depend on values)

    def attention():
        for li in range(cfg.n_layers):
            _ffi.sdpa(q4, dec.k_cache[li], dec.v_cache[li], is_causal=True, need_lse=False, out=o4, kv_lens=kvlen)

    def small():
        # the norms the fold leaves: the first layer's and the final one
        _ffi.rmsnorm(x, dec.layers[0]["n1"], cfg.eps)
        _ffi.rmsnorm(x, dec.norm_f, cfg.eps)

    def head():
        h = _ffi.embedding(dec.embed, tok)
        logits = _ffi.gemm(h, dec.lm_head, trans_b=True)
        _ffi.argmax_lastdim(logits)

    def step():
        dec.length = ctx - 1
        dec._graph_step()

    dec._tok = tok
    dec._tok_out = torch.zeros_like(tok)
    dec._pos = pos.clone()
    dec._kvlen = kvlen.clone()
    n_layer_launch = {"gemm": 4 * cfg.n_layers, "attention": cfg.n_layers, "norm": 2, "embed_head_argmax": 3}
    weights = cfg.n_layers * (W * d + hq * hd * d + 2 * dec.ff * d + dec.ff * d) * 2
    kv = 2 * cfg.n_layers * B * hk * ctx * hd * 2
    head_b = cfg.vocab * d * 2
    small_b = 2 * 2 * B * d * 2
    for name, fn, nbytes in (("gemm", gemms, weights), ("attention", attention, kv), ("norm", small, small_b),
                             ("embed_head_argmax", head, head_b), ("whole_step", step, weights + kv + head_b)):
        if not wanted("decode_step_part", name):
            continue
        # few calls per graph: every whole step moves the device-side position / length counters on
        us = time_us(lambda i: fn(), 1, min(max(2, iters // 4), 16))
        launches = n_layer_launch.get(name, sum(n_layer_launch.values()) + 2)
        T.add("decode_step_part", name, us, bytes_=nbytes, bound="hbm", note=f"{launches} launches per call")


def baseline_sweep(iters=10):
    """The operator sweeps the benchmark configuration names, as rows (no printing): attention
    prefill (batch 8, 32 query heads, 32 or 8 KV heads, S = 1024 / 4096 / 16384) and decode (batch 64,
    caches of 4096 and 32768), the GEMM sweep M in {1, 8, 16, 128, 4096} x four (N, K) plus the batched
    product, and the sampling row ops on the 64 x 128256 logits.  Used by bench.py so that the
    per-operator fractions of peak are measured in the same run as the end-to-end number."""
    global MATCH
    T = Table("", quiet=True)
    saved = MATCH
    try:
        MATCH = "64x128256"
        bench_stream(T, iters)
        torch.cuda.empty_cache()
        MATCH = ""
        bench_sdpa(T, iters)
        torch.cuda.empty_cache()
        for (N, K) in ((4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)):
            for M in (1, 8, 16, 128, 4096):
                MATCH = f"gemm_bf16_tn M{M} N{N} K{K}"
                bench_gemm(T, iters)
            torch.cuda.empty_cache()
        MATCH = "addmm_bias_bf16_tn"
        bench_gemm(T, iters)
        MATCH = "bmm_bf16"
        bench_gemm(T, iters)
    finally:
        MATCH = saved
        torch.cuda.empty_cache()
    keep = ("op", "shape", "us", "bound", "frac", "frac_nominal")
    seen, rows = set(), []
    for r in T.rows:
        key = (r["op"], r["shape"])
        if key not in seen and r["op"] not in ("mm_bf16_nn", "mm_f32_simt"):
            seen.add(key)
            rows.append({k: r[k] for k in keep})
    return rows, T.kind


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="stream,index,decode,sdpa,gemm")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    ap.add_argument("--match", default="", help='only cases whose "op shape" text contains this')
    ap.add_argument("--eager", action="store_true", help="time plain launches instead of a CUDA-graph replay")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("opbench needs a CUDA device")
    global EAGER, MATCH
    EAGER, MATCH = a.eager, a.match
    if a.out:
        Path(a.out).write_text("")
    T = Table(a.out)
    for name in a.only.split(","):
        torch.cuda.synchronize()
        time.sleep(5.0)          # let the part cool between sections: the dense cases run at the power cap
        {"stream": bench_stream, "index": bench_index, "gemm": bench_gemm, "sdpa": bench_sdpa,
         "decode": bench_decode_breakdown}[name](T, a.iters)
        torch.cuda.empty_cache()
    if _ffi.tc_error() != 0:
        print(json.dumps({"error": "a tensor-core pipeline wait timed out"}))


if __name__ == "__main__":
    main()
