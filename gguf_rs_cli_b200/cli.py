"""The command line, in the manner of the reference's (src/main.rs:13-50): the same option
names, meanings and defaults where it has them, with token ids in place of text.

    python -m gguf_rs_cli_b200 -m MODEL_DIR -p 1,2,3 [-p 4,5 ...] [-n 512] [-t 0.7] [--top-k 40]
        [--top-p 0.9] [--rep-penalty 1.1] [-c 8192] [--seed 42] [--stats] [--debug-gpu]
        [--stop-ids 7,9] [--no-eos]

Generated ids go to standard output, one line per prompt, comma separated; everything
else goes to standard error (docs/INFERENCE.md:57 of the reference).  Not taken over:
-s/--system, --smart-context and the interactive chat (text front end), --debug-tokens.
"""
from __future__ import annotations

import argparse
import sys
from typing import List, Optional, Sequence


def parse_ids(text: str) -> List[int]:
    try:
        ids = [int(x) for x in text.replace(",", " ").split()]
    except ValueError:
        raise argparse.ArgumentTypeError(f"token ids must be integers separated by commas or blanks: {text!r}") from None
    if not ids:
        raise argparse.ArgumentTypeError("a prompt needs at least one token id")
    return ids


def parse_stop_ids(text: str) -> List[int]:
    """Stop tokens; an empty string means none (generation then runs to --max-tokens)."""
    return parse_ids(text) if text.strip() else []


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="gguf_rs_cli_b200", description="Llama generation on one B200: token ids in, token ids out")
    src = ap.add_mutually_exclusive_group(required=True)
    src.add_argument("-m", "--model", help="folder with config.json and model.safetensors")
    src.add_argument("--random", metavar="CONFIG_JSON", help="random weights N(0, 0.02) for this config.json")
    ap.add_argument("--weights-seed", type=int, default=0, help="seed of --random weights")
    ap.add_argument("-p", "--prompt-ids", "--prompt", dest="prompts", action="append", type=parse_ids, default=[],
                    help="one request's token ids, e.g. 1,15,27 (repeat for a batch)")
    ap.add_argument("--prompt-ids-file", help="file with one request per line")
    ap.add_argument("-n", "--max-tokens", type=int, default=512)
    ap.add_argument("-t", "--temperature", type=float, default=0.7, help="<= 0 is greedy")
    ap.add_argument("--top-k", type=int, default=40, help="0 turns it off")
    ap.add_argument("--top-p", type=float, default=0.9, help="1 turns it off")
    ap.add_argument("--rep-penalty", type=float, default=1.1, help="1 turns it off; applies to the last 64 generated tokens")
    ap.add_argument("-c", "--ctx-len", type=int, default=8192, help="positions one sequence may hold")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--stats", action="store_true", help="print token throughput after the run")
    ap.add_argument("--gpu", action="store_true", help="accepted for compatibility: this library always runs on the GPU")
    ap.add_argument("--debug-gpu", "--profile", dest="debug_gpu", action="store_true",
                    help="time stamps after each stage of every step (embedding, the first layer's norm, q/k/v, "
                         "attention, output projection, gate+up, down, all layers, head, sampling), one line per step")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--stop-ids", type=parse_stop_ids, default=None,
                    help="further stop tokens, joined with the model's eos ids")
    ap.add_argument("--no-eos", action="store_true",
                    help="leave the model's eos ids out (with no --stop-ids generation runs to --max-tokens)")
    ap.add_argument("--max-batch", type=int, default=64, help="most requests generated together")
    return ap


def main(argv: Optional[Sequence[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    prompts = list(args.prompts)
    if args.prompt_ids_file:
        with open(args.prompt_ids_file) as f:
            prompts += [parse_ids(line) for line in f if line.strip()]
    if not prompts:
        print("error: no prompt given (-p 1,2,3 or --prompt-ids-file)", file=sys.stderr)
        return 2
    from . import native
    from .api import from_random, generate, load
    from .engine.generate import GenerationStats
    try:
        llm = load(args.model, dtype=args.dtype) if args.model else from_random(args.random, args.weights_seed, args.dtype)
    except (ValueError, native.NativeError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    spec = llm.spec
    print(f"Model: {spec.architecture} | layers {len(spec.layers)} | hidden {spec.hidden_size} | vocab {spec.vocab_size}",
          file=sys.stderr)
    # the model's end tokens joined with the caller's, as the reference joins the tokenizer's with the chat
    # template's (src/chat.rs:57-72)
    stops = [] if args.no_eos else list(spec.stop_token_ids)
    stops += [t for t in (args.stop_ids or []) if t not in stops]
    print(f"EOS tokens: {list(stops)}", file=sys.stderr)
    print(f"Params: temp={args.temperature} top_k={args.top_k} top_p={args.top_p} rep_penalty={args.rep_penalty}",
          file=sys.stderr)
    print(f"Context: {min(args.ctx_len, spec.max_position)} tokens | Mode: GPU (CUDA sm_100a, {args.dtype})\n", file=sys.stderr)
    stats = GenerationStats()
    launches0 = native.launch_count()
    try:
        out = generate(llm, prompts, max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k,
                       top_p=args.top_p, rep_penalty=args.rep_penalty, seed=args.seed, stop_token_ids=stops,
                       max_batch=args.max_batch, ctx_len=args.ctx_len, stats=stats, profile=args.debug_gpu)
    except (ValueError, RuntimeError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    for ids in out:
        print(",".join(str(t) for t in ids))
    if args.stats:
        gs = max(stats.decode_seconds, 1e-3)
        print(f"[Stats] prefill: {stats.prompt_tokens} tok in {stats.prefill_seconds * 1000:.0f}ms | generated: "
              f"{stats.generated_tokens} tok in {stats.decode_seconds:.2f}s ({stats.generated_tokens / gs:.1f} tok/s)",
              file=sys.stderr)
    if args.debug_gpu:
        steps = max(stats.decode_steps + stats.batches, 1)
        print(f"[GPU] {native.launch_count() - launches0} kernel launches in {steps} steps; decode "
              f"{stats.decode_seconds * 1000 / max(stats.decode_steps, 1):.3f} ms/step", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
