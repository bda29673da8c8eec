"""Batched greedy / sampled generation of a HuggingFace causal LM under the kuiops dispatch mode.

The command-line surface of the reference's driver (infer.py:289-357 there): a positional prompt
or ``--prompts FILE``, ``--batch``, ``--max-new-tokens``, ``--temperature``, ``--print``,
``--no-kuiper``, ``--timing``, ``--verify``, ``--verify-tol``.  The reference hard-codes a model
that it downloads; here the model comes from a local directory (``--model-dir``, a HuggingFace
checkpoint with or without a tokenizer) or is built from a named shape with random weights
(``--shape``), which is all that can be exercised without a network.  Without a tokenizer a
prompt is mapped to ids byte by byte and responses are printed as ids.

``--timing`` prints the prefill / decode split of the reference's minimal script
(infer_minimal.py:68-76: prefill = a generation of one token, decode = the rest divided by the
remaining tokens) instead of a profiler table.
"""
import argparse
import sys
import time
from contextlib import nullcontext
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
import kuipy  # noqa: E402

DEFAULT_BATCH = 8
SHAPES = {
    # name: (model_type, config keyword arguments)
    "tiny": ("llama", dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, vocab_size=1000, max_position_embeddings=512)),
    "qwen2.5-0.5b": ("qwen2", dict(hidden_size=896, intermediate_size=4864, num_hidden_layers=24, num_attention_heads=14,
                                   num_key_value_heads=2, vocab_size=151936, max_position_embeddings=4096,
                                   tie_word_embeddings=True, rope_theta=1e6)),
    "llama3-8b": ("llama", dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                                num_key_value_heads=8, vocab_size=128256, max_position_embeddings=8192, rope_theta=5e5,
                                rms_norm_eps=1e-5)),
    "gpt2-small": ("gpt2", dict(n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257, n_positions=1024)),
}


def load_model(model_dir, shape, device, dtype, seed=0):
    """(model, tokenizer or None).  A directory wins over a shape."""
    from transformers import AutoConfig, AutoModelForCausalLM
    tok = None
    if model_dir:
        model = AutoModelForCausalLM.from_pretrained(model_dir, dtype=dtype, local_files_only=True)
        try:
            from transformers import AutoTokenizer
            tok = AutoTokenizer.from_pretrained(model_dir, local_files_only=True, padding_side="left")
            if tok.pad_token_id is None:
                tok.pad_token = tok.eos_token
        except (OSError, ValueError):
            tok = None
    else:
        kind, kw = SHAPES[shape]
        cfg = AutoConfig.for_model(kind, **kw)
        torch.manual_seed(seed)
        model = AutoModelForCausalLM.from_config(cfg, dtype=dtype)
    return model.to(device).eval(), tok


def encode(prompts, tok, vocab, device):
    """Left-padded ids and attention mask of a batch of prompts."""
    if tok is not None:
        enc = tok(prompts, return_tensors="pt", padding=True)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device), tok.pad_token_id
    rows = [[b % vocab for b in p.encode("utf-8")] or [0] for p in prompts]
    width = max(len(r) for r in rows)
    ids = torch.zeros((len(rows), width), dtype=torch.int64)
    mask = torch.zeros_like(ids)
    for i, r in enumerate(rows):
        ids[i, width - len(r):] = torch.tensor(r)
        mask[i, width - len(r):] = 1
    return ids.to(device), mask.to(device), 0


def generate_batch(model, tok, prompts, *, max_new_tokens=64, temperature=0.7, pad_to_multiple=DEFAULT_BATCH,
                   use_kuiper=True, timing=False, verify=False, verify_tol=2e-2, out=None):
    """Mirror of the reference's generate_batch (infer.py:78-176): pads the batch with copies of the
    last prompt, runs ``model.generate`` under ``KuiperMode`` and prints the same throughput line.
    Returns (responses, verify_ok)."""
    out = out or sys.stdout
    device = next(model.parameters()).device
    real_n = len(prompts)
    padded = list(prompts)
    while len(padded) % max(1, pad_to_multiple):
        padded.append(prompts[-1])
    ids, mask, pad_id = encode(padded, tok, model.config.vocab_size, device)
    on_gpu = device.type == "cuda"
    if verify and not (kuipy.is_available() and on_gpu):
        print("[verify] kuiops unavailable on this device: nothing to verify.", file=sys.stderr)
        verify = False
    if kuipy.is_available() and use_kuiper and on_gpu:
        ctx, tag = kuipy.KuiperMode(verify=verify, verify_tol=verify_tol), ("kuiper+verify" if verify else "kuiper")
    else:
        ctx, tag = nullcontext(), "torch"
    if verify:
        kuipy.reset_verify()
    kw = dict(input_ids=ids, attention_mask=mask, temperature=temperature if temperature > 0 else None,
              do_sample=temperature > 0, pad_token_id=pad_id)

    def run(n_new):
        if on_gpu:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        with ctx, torch.no_grad():
            o = model.generate(max_new_tokens=n_new, min_new_tokens=n_new, **kw)
        if on_gpu:
            torch.cuda.synchronize()
        return o, time.perf_counter() - t0

    prefill_s = None
    if timing:
        run(1)                                  # warm caches and allocator
        _, prefill_s = run(1)
    outputs, elapsed = run(max_new_tokens)
    new_tokens = outputs[:, ids.shape[-1]:]
    n_new = new_tokens.shape[-1]
    if tok is not None:
        decoded = tok.batch_decode(new_tokens, skip_special_tokens=True)[:real_n]
    else:
        decoded = [" ".join(str(int(t)) for t in row) for row in new_tokens[:real_n]]
    print(f"[batched generate / {tag}] {real_n} prompts (padded to {len(padded)}), {n_new} new tokens each -> "
          f"{elapsed:.2f}s ({n_new * real_n / elapsed:.1f} real tok/s, {n_new * len(padded) / elapsed:.1f} kernel tok/s)", file=out)
    if timing and prefill_s is not None and n_new > 1:
        per_tok = (elapsed - prefill_s) / (n_new - 1)
        print(f"[timing] prefill {prefill_s * 1e3:.1f} ms ({ids.numel() / prefill_s:.0f} tok/s), "
              f"decode {per_tok * 1e3:.2f} ms/token ({len(padded) / per_tok:.0f} tok/s)", file=out)
    ok = True
    if verify:
        ok = kuipy.print_verify_report(out, tol=verify_tol) is not False
    return decoded, ok


def build_parser():
    ap = argparse.ArgumentParser(description="Batched causal-LM inference through kuiops")
    ap.add_argument("prompt", nargs="?", default=None, help="single prompt (replicated to fill the batch)")
    ap.add_argument("--prompts", type=Path, default=None, help="file with one prompt per line")
    ap.add_argument("--batch", type=int, default=DEFAULT_BATCH, help=f"batch size to pad up to (default {DEFAULT_BATCH})")
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--print", dest="show", action="store_true", help="print every response")
    ap.add_argument("--no-kuiper", dest="use_kuiper", action="store_false", help="stock PyTorch, for A/B comparison")
    ap.set_defaults(use_kuiper=True)
    ap.add_argument("--timing", action="store_true", help="print the prefill / decode split")
    ap.add_argument("--verify", action="store_true", help="run every dispatched op through PyTorch too and report divergences")
    ap.add_argument("--verify-tol", type=float, default=2e-2)
    ap.add_argument("--model-dir", type=Path, default=None, help="local HuggingFace checkpoint directory")
    ap.add_argument("--shape", default="qwen2.5-0.5b", choices=sorted(SHAPES), help="random-weight model when no --model-dir")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    return ap


def main(argv=None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    if args.prompt and args.prompts:
        ap.error("pass either a positional prompt or --prompts FILE, not both")
    if args.verify and not args.use_kuiper:
        ap.error("--verify requires the kuiops kernels; do not combine it with --no-kuiper")
    if args.prompts is not None:
        prompts = [ln.strip() for ln in args.prompts.read_text().splitlines() if ln.strip()]
        if not prompts:
            print(f"[infer] no prompts found in {args.prompts}", file=sys.stderr)
            return 1
    elif args.prompt is not None:
        prompts = [args.prompt]
    else:
        prompts = [f"Synthetic prompt number {i}: continue the sequence." for i in range(args.batch)]
        print(f"[infer] no prompts given: using {len(prompts)} synthetic prompts.\n")
    model, tok = load_model(args.model_dir, args.shape, args.device, getattr(torch, args.dtype))
    responses, ok = generate_batch(model, tok, prompts, max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                                   pad_to_multiple=args.batch, use_kuiper=args.use_kuiper, timing=args.timing,
                                   verify=args.verify, verify_tol=args.verify_tol)
    show_n = len(responses) if args.show else min(3, len(responses))
    for i in range(show_n):
        print("\n" + "-" * 70)
        print(f"Prompt {i}:  {prompts[i]}")
        print(f"Response:  {responses[i].strip()}")
    if show_n < len(responses):
        print(f"\n... ({len(responses) - show_n} more, pass --print to see all)")
    return 0 if ok else 2


if __name__ == "__main__":
    sys.exit(main())
