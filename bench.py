#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-3.1-8B shape with random bf16 weights on
one B200.  Prints one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--layers L] [--batch B] [--no-points] [--prompt-steps 128,256] [--shape 8b|1b|13b]

`value` is decoded tokens a second at batch 8 after 512-token prompts, timed on the
device with CUDA events around K decode steps (each step: index arrays host to
device, the model, sampling, sampled ids device to host).  `e2e` is the same through
the Python entry point `generate()`, host token ids in and out.  `prefill` is one
step of 2,048 tokens; `points` are decode at batch 1 and 64; `roofline` is the bytes a
decode step has to read (every weight once, the cache of the live requests) over its
time, against the measured copy bandwidth.  The weights (15 GB) are far larger than
L2, so consecutive steps cannot reuse cached inputs.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 32, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
    "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 8192, "tie_word_embeddings": False, "hidden_act": "silu",
}
# The two further workloads: unequal prompts through generate(), then 256 decode steps.
SHAPE_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 16, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 8192, "tie_word_embeddings": True, "hidden_act": "silu",
}
SHAPE_13B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 40, "hidden_size": 5120,
    "num_attention_heads": 40, "num_key_value_heads": 40, "head_dim": 128, "intermediate_size": 13824,
    "vocab_size": 32000, "rope_theta": 10000.0, "rope_scaling": None,
    "rms_norm_eps": 1e-5, "max_position_embeddings": 4096, "tie_word_embeddings": False, "hidden_act": "silu",
}
WORKLOADS = {"1b": (SHAPE_1B, "llama-3.2-1b-shape", 16, 64, 1024), "13b": (SHAPE_13B, "llama-2-13b-shape", 32, 128, 2048)}
WORKLOAD_STEPS = 256
CONTEXT = 8192
PROMPT = 512
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
        out = {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
        if raw.get("bf16_tflops_sustained"):
            out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
        return out
    except Exception:
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def mark(self):
        return time.time()

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, t0, t1):
        rows = [r for t, r in self.rows if t0 <= t <= t1 and len(r) >= 6] or [r for _, r in self.rows if len(r) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(int(r[0]) for r in rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None,
                "sm_max_mhz": int(rows[0][1]) if rows[0][1].isdigit() else None, "reasons": reasons, "samples": len(rows)}


def weight_bytes(cfg, layers):
    """Bytes of weights a decode step reads: every layer, the final norm and the head (for a tied head the
    embedding table, read once as the head); the embedding rows of the step's tokens are negligible."""
    E, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh * hd * E + 2 * nkv * hd * E + E * nh * hd + 3 * F * E + 2 * E) * 2
    return layers * per_layer + (V * E + E) * 2


def kv_bytes_per_token(cfg, layers):
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, layers, T):
    E, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2 * T * layers * (nh * hd * E + 2 * nkv * hd * E + E * nh * hd + 3 * F * E)
    attn = layers * 4 * nh * hd * T * (T + 1) // 2
    return linear + attn + 2 * V * E


def measure_decode(llm, batch, steps, warmup, cfg, sampling=None):
    """K decode steps at `batch` after 512-token prompts.  Returns (tokens/s, ms/step,
    launches per step, context at the middle of the timed steps)."""
    import torch
    from gguf_rs_cli_b200 import native
    from gguf_rs_cli_b200.sampling import SamplingParams, stream_key
    g = torch.Generator().manual_seed(batch)
    prompts = [torch.randint(0, cfg["vocab_size"], (PROMPT,), generator=g).tolist() for _ in range(batch)]
    backend = llm.backend(n_tokens=64 * CONTEXT, n_slots=64, max_len=CONTEXT)
    params = SamplingParams(**(sampling or {"temperature": 0.0}))
    keys = [stream_key(0, i) for i in range(batch)]
    slots = [backend.open() for _ in range(batch)]
    toks = backend.run(slots, prompts, keys, params)
    for _ in range(warmup):
        toks = backend.run(slots, [[t] for t in toks], keys, params)
    torch.cuda.synchronize()
    n0 = native.launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    # as the generation loop drives it: each step is launched, fed on the device, before the tokens of the step in
    # front of it are read, so the device does not wait for the host between steps
    pending = backend.begin(slots, [[t] for t in toks], keys, params)
    for i in range(steps):
        ahead = backend.begin_after(pending) if i + 1 < steps else None
        toks = backend.finish(pending)
        if i + 1 < steps:
            pending = ahead if ahead is not None else backend.begin(slots, [[t] for t in toks], keys, params)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launches = (native.launch_count() - n0) // steps
    for s in slots:
        backend.close(s)
    ctx_mid = PROMPT + warmup + steps // 2
    return batch * 1000.0 / ms, ms, launches, ctx_mid


def measure_prefill(llm, cfg, layers, reps=3, tokens=PREFILL_TOKENS):
    """Milliseconds of one prompt step of `tokens` tokens (one sequence, logits at its last place), best of reps."""
    import torch
    from gguf_rs_cli_b200.engine.step import Entry
    eng = llm.engine(n_tokens=64 * CONTEXT, n_slots=64, max_len=CONTEXT)
    g = torch.Generator().manual_seed(7)
    toks = torch.randint(0, cfg["vocab_size"], (tokens,), generator=g).tolist()
    best = None
    for i in range(reps + 1):
        s = eng.open()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step([Entry(s, toks, [tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        eng.close(s)
        if i:                                       # the first run warms up
            ms = a.elapsed_time(b)
            best = ms if best is None else min(best, ms)
    return best


def measure_e2e(llm, cfg, batch, steps, warmup):
    """Through generate(): host ids in, host ids out.  Decode tokens a second from the
    loop's own clock (synchronised on both sides of every step).  A short untimed call
    comes first: it is the warm-up (the first steps of a batch size build its graph)."""
    import torch
    from gguf_rs_cli_b200.api import generate
    from gguf_rs_cli_b200.engine.generate import GenerationStats
    g = torch.Generator().manual_seed(100 + batch)
    prompts = [torch.randint(0, cfg["vocab_size"], (PROMPT,), generator=g).tolist() for _ in range(batch)]
    backend = llm.backend(n_tokens=64 * CONTEXT, n_slots=64, max_len=CONTEXT)
    h0, d0 = backend.h2d_bytes, backend.d2h_bytes
    generate(llm, prompts, max_tokens=warmup + 2, temperature=0.0, stop_token_ids=[], max_batch=64, ctx_len=CONTEXT)
    h0, d0 = backend.h2d_bytes, backend.d2h_bytes
    stats = GenerationStats()
    out = generate(llm, prompts, max_tokens=steps, temperature=0.0, stop_token_ids=[], max_batch=64, ctx_len=CONTEXT,
                   stats=stats)
    assert all(len(o) == steps for o in out)
    n_steps = stats.decode_steps + 1
    tok_s = batch * stats.decode_steps / max(stats.decode_seconds, 1e-9)
    return tok_s, (backend.h2d_bytes - h0) // n_steps, (backend.d2h_bytes - d0) // n_steps


def run_workload(name, layers_arg, pk):
    """One of the further workloads, through the Python entry point: a batch of unequal prompts (lengths uniform
    in the workload's range, seeded) in one step, then 256 decode steps with every sequence alive.  One JSON line:
    decode tokens a second (the loop's own clock, synchronised around every step), the prompt step, and the
    decode step's bytes (weights once, the cache of the live sequences at the middle step) over its time."""
    import torch
    from gguf_rs_cli_b200.api import from_random, generate
    from gguf_rs_cli_b200.engine.generate import GenerationStats
    cfg, model_name, n_prompts, lo, hi = WORKLOADS[name]
    cfg = dict(cfg)
    full_layers = cfg["num_hidden_layers"]
    layers = full_layers if layers_arg is None else layers_arg
    cfg["num_hidden_layers"] = layers
    llm = from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(lo, hi + 1, (n_prompts,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    ctx = cfg["max_position_embeddings"]
    sampler = ClockSampler()
    sampler.start()
    best = None
    for rep in range(3):                                  # the first pass warms up (kernels, graphs of this batch size)
        stats = GenerationStats()
        t0 = sampler.mark()
        out = generate(llm, prompts, max_tokens=WORKLOAD_STEPS, temperature=0.0, stop_token_ids=[], max_batch=64,
                       ctx_len=ctx, stats=stats)
        t1 = sampler.mark()
        assert all(len(o) == WORKLOAD_STEPS for o in out)
        if rep and (best is None or stats.decode_seconds < best[0].decode_seconds):
            best = (stats, t0, t1)
    sampler.stop()
    stats, t0, t1 = best
    ms = stats.decode_seconds * 1e3 / stats.decode_steps
    mid_tokens = sum(lens) + n_prompts * (WORKLOAD_STEPS // 2)
    step_bytes = weight_bytes(cfg, layers) + mid_tokens * kv_bytes_per_token(cfg, layers)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = sum(prefill_flops(cfg, layers, n) for n in lens)
    line = {
        "metric": f"{model_name} decode tok/s @ batch {n_prompts} (prompts of {lo} to {hi} tokens, {WORKLOAD_STEPS} steps)",
        "value": round(n_prompts * 1000.0 / ms, 2), "unit": "tokens/s", "n_gpus": 1, "steps": stats.decode_steps, "warmup": 1,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random weights N(0,0.02)", "impl": "ours",
        "config": {"model": model_name, "layers": layers, "layers_full": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": n_prompts,
                   "seq_len": ctx, "prompt_tokens": sum(lens), "parallelism": "single-gpu", "peaks": pk["source"],
                   "timing": "through generate(), host ids in and out, synchronised around every step"},
        "clocks": sampler.summary(t0, t1),
        "prefill": {"value": round(stats.prompt_tokens / stats.prefill_seconds, 1), "tokens": stats.prompt_tokens,
                    "ms": round(stats.prefill_seconds * 1e3, 3),
                    "frac": round(flops / stats.prefill_seconds / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": step_bytes},
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (profiles)")
    ap.add_argument("--shape", default="8b", choices=["8b", "1b", "13b"],
                    help="8b: the headline line; 1b, 13b: the further workloads (unequal prompts, 256 decode steps)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1/64, prefill and e2e")
    ap.add_argument("--temperature", type=float, default=0.0, help="sampling of the device-timed decode steps (default greedy)")
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--rep-penalty", type=float, default=1.0)
    ap.add_argument("--prompt-steps", default="", help="also time prompt steps of these many tokens, e.g. 128,256,512")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust/Vulkan program: pip finds neither "
                          "setup.py nor pyproject.toml, and the image has no cargo, rustc or Vulkan loader"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)
    if args.shape != "8b":
        return run_workload(args.shape, args.layers, peaks())
    if args.layers is None:
        args.layers = SHAPE_8B["num_hidden_layers"]

    import torch
    from gguf_rs_cli_b200 import native
    from gguf_rs_cli_b200.api import from_random
    cfg = dict(SHAPE_8B)
    full_layers = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    llm = from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    torch.cuda.synchronize()

    sampler = ClockSampler()
    sampler.start()
    t0 = sampler.mark()
    sampling = {"temperature": args.temperature, "top_k": args.top_k, "top_p": args.top_p, "rep_penalty": args.rep_penalty}
    tok_s, ms, launches, ctx_mid = measure_decode(llm, args.batch, args.steps, warmup, cfg, sampling)
    t1 = sampler.mark()
    clocks = sampler.summary(t0, t1)

    wbytes, kvb = weight_bytes(cfg, args.layers), kv_bytes_per_token(cfg, args.layers)
    step_bytes = wbytes + args.batch * ctx_mid * kvb
    achieved = step_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": f"Llama-3.1-8B decode tok/s @ batch {args.batch} ({PROMPT}-token prompts)", "value": round(tok_s, 2), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights N(0,0.02)",
        "impl": "ours",
        "config": {"model": "llama-3.1-8b-shape", "layers": args.layers, "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
                   "seq_len": CONTEXT, "prompt_len": PROMPT, "parallelism": "single-gpu",
                   "l2": f"inputs ({wbytes / 1e9:.1f} GB of weights per step) exceed L2", "peaks": pk["source"]},
        "clocks": clocks, "gpu_launches": launches * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": step_bytes},
    }
    if not args.no_points:
        # the end-to-end figure right after the device-timed one (the same state of the device), then the rest
        e_tok_s, h2d, d2h = measure_e2e(llm, cfg, args.batch, args.steps, warmup)
        line["e2e"] = {"value": round(e_tok_s, 2), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                       "d2h_bytes_per_step": int(d2h)}
        pms = measure_prefill(llm, cfg, args.layers)
        flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
        line["prefill"] = {"value": round(PREFILL_TOKENS * 1000.0 / pms, 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                           "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        points = {}
        for b in (1, 64):
            p_steps = max(8, args.steps // 2)
            p_tok_s, p_ms, _, p_ctx = measure_decode(llm, b, p_steps, warmup, cfg)
            points[f"decode_b{b}"] = round(p_tok_s, 2)
            points[f"decode_b{b}_ms"] = round(p_ms, 4)
            points[f"decode_b{b}_frac"] = round((wbytes + b * p_ctx * kvb) / (p_ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        line["points"] = points
    if args.prompt_steps:
        # short prompt steps: bound by the weights they stream (once) rather than by the tensor rate
        extra = {}
        for t in [int(x) for x in args.prompt_steps.split(",") if x.strip()]:
            t_ms = measure_prefill(llm, cfg, args.layers, reps=5, tokens=t)
            extra[f"prompt_{t}_ms"] = round(t_ms, 3)
            extra[f"prompt_{t}_x_weights"] = round(t_ms * 1e-3 / (wbytes / (pk["hbm_gbs"] * 1e9)), 2)
        line.setdefault("points", {}).update(extra)
    sampler.stop()
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
