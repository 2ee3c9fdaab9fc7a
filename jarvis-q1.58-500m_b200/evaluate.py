"""Corpus perplexity, single-prompt generation and an interactive prompt on the sm_100a modules.

Command-line twin of the reference's jarvis_engine/evaluate_jarvis.py (flags of its parse_args, :55-90):

    python -m jarvis_b200.evaluate --ckpt model.pt --eval-file holdout.txt --num-windows 200 --seq-len 256
    python -m jarvis_b200.evaluate --ckpt model.jarvis-tbin --prompt "..." --max_new_tokens 64
    python -m jarvis_b200.evaluate --ckpt model.pt -i

What is kept: the window selection and statistics of evaluate_corpus (:323-377: consecutive windows when the
corpus is long enough, else seeded random starts; loss of `model(x, targets=y)` per window, mean / stdev /
exp(mean)), the generation loop of generate_streaming (:186-268: state reset, context = last 256 tokens re-run
every step, stop at the end-of-text token) and the REPL commands (/reset, /info, /quit).  What differs: the
sampling filter runs in `jb200_sample` (uniform numbers from a seeded torch generator); `--stateful` decodes
with the carried recurrent state (one token per step through the CUDA-graphed step) instead of re-running the
window; checkpoints may be a training `.pt` (`model_state_dict`), a packed state dict or a `.jarvis-tbin`
container; corpora may be text (needs the GPT-2 encoding of `tiktoken`, which must already be cached: there is
no download here) or token ids (`.npy`, `.pt`, or whitespace-separated integers in a `.ids` file).
"""
from __future__ import annotations

import argparse
import math
import os
import statistics
import sys
import time

import torch

CONTEXT_WINDOW = 256   # the reference re-runs at most this many trailing tokens per generated token


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Jarvis evaluation / generation on the sm_100a kernels")
    p.add_argument("--interactive", "-i", action="store_true", help="prompt loop on the terminal")
    p.add_argument("--prompt", type=str, default=None, help="generate once from this prompt")
    p.add_argument("--max_new_tokens", type=int, default=128)
    p.add_argument("--temperature", type=float, default=0.7, help="0 = greedy")
    p.add_argument("--top_k", type=int, default=50, help="1..1024")
    p.add_argument("--top_p", type=float, default=0.9, help="1.0 disables the nucleus cut")
    p.add_argument("--ckpt", type=str, default="ckpt_step_0004209.pt")
    p.add_argument("--eval-file", type=str, default="fresh_holdout.txt")
    p.add_argument("--train-file", type=str, default="data.txt")
    p.add_argument("--num-windows", type=int, default=200)
    p.add_argument("--seq-len", type=int, default=256)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--skip-train-eval", action="store_true")
    p.add_argument("--skip-gen", action="store_true")
    p.add_argument("--stateful", action="store_true", help="decode with the carried recurrent state (not the 256-token re-run)")
    p.add_argument("--layers", type=int, default=24)
    p.add_argument("--d-model", type=int, default=1024)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--vocab", type=int, default=50257)
    return p.parse_args(argv)


# ---- tokens ---------------------------------------------------------------------------------------
class IdTokenizer:
    """Stand-in when no text encoding is available: text is a list of integers separated by spaces."""
    eot_token = None

    def encode(self, text):
        return [int(t) for t in text.split()]

    def decode(self, ids):
        return " ".join(str(i) for i in ids)


def get_tokenizer():
    try:
        import tiktoken
        return tiktoken.get_encoding("gpt2")
    except Exception as exc:  # not installed, or its vocabulary is not cached and cannot be fetched
        print(f"[evaluate] GPT-2 encoding unavailable ({type(exc).__name__}); prompts are read as token ids", file=sys.stderr)
        return IdTokenizer()


def load_token_file(path: str, enc) -> torch.Tensor:
    """Token ids of a corpus file: .npy / .pt hold ids, .ids holds integers as text, anything else is text."""
    if not os.path.exists(path):
        raise FileNotFoundError(f"corpus file '{path}' does not exist (no fallback to another corpus)")
    ext = os.path.splitext(path)[1].lower()
    if ext == ".npy":
        import numpy as np
        return torch.from_numpy(np.load(path).astype("int64")).view(-1)
    if ext == ".pt":
        return torch.load(path, map_location="cpu").to(torch.int64).view(-1)
    with open(path, "r", encoding="utf-8", errors="ignore") as fh:
        text = fh.read()
    if ext == ".ids":
        return torch.tensor([int(t) for t in text.split()], dtype=torch.int64)
    return torch.tensor(enc.encode(text), dtype=torch.int64)


# ---- model ----------------------------------------------------------------------------------------
def load_model(ckpt_path: str, *, vocab=50257, d_model=1024, n_layers=24, n_heads=16, device="cuda"):
    """Build the sm_100a `Jarvis` and load `ckpt_path`: a training checkpoint ({"model_state_dict": ...},
    keys possibly prefixed `_orig_mod.`), a packed state dict (`*.packed_weight` / `*.alpha`) or a
    `.jarvis-tbin` container.  Strict: every key must match.  -> (model, trained step or None)."""
    from . import checkpoint, modules
    if not os.path.exists(ckpt_path):
        raise FileNotFoundError(f"checkpoint '{ckpt_path}' not found")
    model = modules.Jarvis(vocab_size=vocab, d_model=d_model, n_layers=n_layers, n_heads=n_heads,
                           max_seq_len=CONTEXT_WINDOW).to(device).eval()
    step = None
    if ckpt_path.endswith(".jarvis-tbin"):
        packed, _ = checkpoint.read_tbin(ckpt_path)
        checkpoint.load_packed_state_dict(model, packed)
    else:
        blob = torch.load(ckpt_path, map_location="cpu", weights_only=False)
        sd = blob["model_state_dict"] if isinstance(blob, dict) and "model_state_dict" in blob else blob
        step = blob.get("step") if isinstance(blob, dict) else None
        sd = {(k[len("_orig_mod."):] if k.startswith("_orig_mod.") else k): v for k, v in sd.items()}
        if any(k.endswith(".packed_weight") for k in sd):
            checkpoint.load_packed_state_dict(model, sd)
        else:
            missing, unexpected = model.load_state_dict(sd, strict=True)
            if missing or unexpected:
                raise RuntimeError(f"checkpoint mismatch: missing={missing}, unexpected={unexpected}")
    return model, step


def model_info(model, ckpt_path: str) -> str:
    n, text = model.param_count()
    st = model.get_backend_status()
    dev = model.tok_emb.weight.device
    lines = [f"checkpoint        {ckpt_path}",
             f"parameters        {n:,} ({text})",
             f"attention / MoE   {st['attn_backend']} ({st['attn_cuda_blocks']}) / {st['moe_backend']} ({st['moe_cuda_blocks']})",
             f"device            {torch.cuda.get_device_name(dev) if dev.type == 'cuda' else 'cpu'}",
             f"memory            {torch.cuda.memory_allocated() / 2**30:.2f} GiB allocated" if dev.type == "cuda" else "memory            -",
             f"liquid states     {sum(h is not None for h in model._h_states)}/{len(model.blocks)} layers, position {model._token_pos}"]
    return "\n".join(lines)


# ---- corpus evaluation ------------------------------------------------------------------------------
def window_starts(n_tokens: int, num_windows: int, seq_len: int, seed: int):
    """evaluate_corpus' choice (evaluate_jarvis.py:337-345): back-to-back windows when the corpus holds
    num_windows * (seq_len + 1) tokens, else num_windows seeded random starts in [0, n_tokens - seq_len - 1)."""
    if n_tokens < seq_len + 1:
        raise ValueError(f"corpus has {n_tokens} tokens, fewer than the {seq_len + 1} one window needs")
    if n_tokens >= num_windows * (seq_len + 1):
        return [i * seq_len for i in range(num_windows)]
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(0, n_tokens - seq_len - 1, (num_windows,), generator=g).tolist()


@torch.no_grad()
def evaluate_corpus(model, tokens: torch.Tensor, num_windows=200, seq_len=256, seed=42, label="HOLDOUT"):
    """Mean / stdev of the per-window loss `model(x, targets=y)` and exp(mean) (evaluate_jarvis.py:323-377)."""
    dev = model.tok_emb.weight.device
    tokens = tokens.to(dev)
    losses, bad = [], False
    for s in window_starts(int(tokens.numel()), num_windows, seq_len, seed):
        x = tokens[s:s + seq_len].unsqueeze(0)
        y = tokens[s + 1:s + seq_len + 1].unsqueeze(0)
        _, loss = model(x, targets=y, persist_state=False)
        v = float(loss)
        bad = bad or math.isnan(v) or math.isinf(v)
        losses.append(v)
    mean = statistics.mean(losses)
    return {"label": label, "corpus_total_tokens": int(tokens.numel()), "windows_evaluated": len(losses),
            "tokens_evaluated": num_windows * seq_len, "mean_loss": mean,
            "std_loss": statistics.stdev(losses) if len(losses) > 1 else 0.0,
            "perplexity": math.exp(min(mean, 100.0)), "has_nan_inf": bad}


# ---- generation -------------------------------------------------------------------------------------
@torch.no_grad()
def generate(model, prompt_ids, max_new_tokens=128, temperature=0.7, top_k=50, top_p=0.9, eot_token=None, seed=0,
             stateful=False, on_token=None):
    """Token ids generated after `prompt_ids`.  stateful=False re-runs the trailing CONTEXT_WINDOW tokens for
    every new token with `persist_state=False`, as generate_streaming does (evaluate_jarvis.py:216-225);
    stateful=True prefills once and then advances the carried state one token at a time."""
    from . import ops
    dev = model.tok_emb.weight.device
    model.reset_state()
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    greedy = temperature is None or temperature <= 0.0
    ids = list(prompt_ids) if len(prompt_ids) else ([eot_token] if eot_token is not None else [0])
    out = []

    def draw(row):       # row: (1, V) logits
        u = None if greedy else torch.rand((1,), dtype=torch.float32, device=dev, generator=gen)
        return int(ops.sample(row, u, temperature=0.0 if greedy else temperature, top_k=top_k, top_p=top_p))

    state, pos = None, 0
    for _ in range(max_new_tokens):
        if stateful:
            feed = ids if state is None else ids[-1:]
            logits, state = model.step(torch.tensor([feed], dtype=torch.int64, device=dev), positions=pos, state=state,
                                       max_position=len(prompt_ids) + max_new_tokens + 1)
            pos += len(feed)
        else:
            ctx = torch.tensor([ids[-CONTEXT_WINDOW:]], dtype=torch.int64, device=dev)
            logits, _ = model(ctx, persist_state=False)
        tok = draw(logits[:, -1, :])
        if eot_token is not None and tok == eot_token:
            break
        out.append(tok)
        ids.append(tok)
        if on_token:
            on_token(out)
    model.reset_state()
    return out


def generate_streaming(model, enc, prompt_text, args, out=sys.stdout):
    printed = [0]

    def show(ids):
        text = enc.decode(ids)
        out.write(text[printed[0]:])
        out.flush()
        printed[0] = len(text)

    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    ids = generate(model, enc.encode(prompt_text), args.max_new_tokens, args.temperature, args.top_k, args.top_p,
                   getattr(enc, "eot_token", None), args.seed, args.stateful, on_token=show)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    out.write(f"\n[{len(ids)} tokens, {dt:.3f} s, {len(ids) / max(dt, 1e-5):.1f} tok/s]\n")
    return enc.decode(ids)


def interactive(model, enc, args, ckpt_path):
    print("commands: /reset  /info  /quit")
    while True:
        try:
            line = input("Jarvis> ").strip()
        except (EOFError, KeyboardInterrupt):
            break
        if not line:
            continue
        if line.lower() in ("/quit", "/exit"):
            break
        if line.lower() == "/reset":
            model.reset_state()
            print("state cleared")
        elif line.lower() == "/info":
            print(model_info(model, ckpt_path))
        else:
            generate_streaming(model, enc, line, args)


def main(argv=None):
    args = parse_args(argv)
    torch.manual_seed(args.seed)
    enc = get_tokenizer()
    model, step = load_model(args.ckpt, vocab=args.vocab, d_model=args.d_model, n_layers=args.layers, n_heads=args.heads)
    print(model_info(model, args.ckpt) + (f"\ntrained step      {step}" if step is not None else ""))
    if args.interactive:
        return interactive(model, enc, args, args.ckpt)
    if args.prompt:
        generate_streaming(model, enc, args.prompt, args)
        return
    reports = [evaluate_corpus(model, load_token_file(args.eval_file, enc), args.num_windows, args.seq_len, args.seed, "HOLDOUT")]
    if not args.skip_train_eval:
        reports.append(evaluate_corpus(model, load_token_file(args.train_file, enc), args.num_windows, args.seq_len,
                                       args.seed, "TRAIN"))
    for r in reports:
        print(f"{r['label']:8s} windows {r['windows_evaluated']}  loss {r['mean_loss']:.4f} +- {r['std_loss']:.4f}  "
              f"ppl {r['perplexity']:.2f}{'  NaN/Inf seen' if r['has_nan_inf'] else ''}")
    if len(reports) == 2:
        print(f"generalisation gap (holdout - train loss): {reports[0]['mean_loss'] - reports[1]['mean_loss']:+.4f}")
    return reports


if __name__ == "__main__":
    main()
