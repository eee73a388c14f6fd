#!/usr/bin/env python3
"""Measurement: decode and prompt throughput of Gemma-2 2B sizes with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch B] [--ctx C] [--layers L]

A "step" is one decode step of the whole batch.  The timed region is K decode steps that end
at context length C (default 8192, the benchmark context of the 2B configuration), timed on
the device with CUDA events; `value` is decoded tokens per second.  `e2e` is the same steps
through the public entry point (`Engine.generate_from_ids` on conversations that hold the
context): every step uploads which slots run from pinned memory and brings the sampled ids
back to the host, where the loop reads them one step late.  `prefill` is one prompt of 2,048 tokens.  `roofline` relates the bytes a decode
step must read (every weight once, and the cache of the live sequences) to its time.
`points` holds decoding at batch 1 and 64.  One JSON line is printed.

Random weights are made on the device; the cache of the decode measurements is filled with
random keys and values instead of being computed by a prompt (a decode step reads the same
bytes either way), and says so under config.cache_fill.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Gemma-2 2B layer sizes
GEMMA2_2B = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2", num_hidden_layers=26, hidden_size=2304,
    num_attention_heads=8, num_key_value_heads=4, head_dim=256, intermediate_size=9216,
    vocab_size=256000, rope_theta=10000.0, sliding_window=4096, max_position_embeddings=8192,
    query_pre_attn_scalar=256, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
    rms_norm_eps=1e-6, tie_word_embeddings=True)
# Gemma-2 9B and 27B layer sizes; not part of the default line
GEMMA2_9B = dict(GEMMA2_2B, num_hidden_layers=42, hidden_size=3584, num_attention_heads=16,
                 num_key_value_heads=8, head_dim=256, intermediate_size=14336, query_pre_attn_scalar=256)
GEMMA2_27B = dict(GEMMA2_2B, num_hidden_layers=46, hidden_size=4608, num_attention_heads=32,
                  num_key_value_heads=16, head_dim=128, intermediate_size=36864, query_pre_attn_scalar=144)
MODELS = {"2b": GEMMA2_2B, "9b": GEMMA2_9B, "27b": GEMMA2_27B}
FULL_LAYERS = 26
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            out, found = dict(FALLBACK_PEAKS), 0

            def look(node):            # the keys may sit at the top or one level down
                nonlocal found
                if not isinstance(node, dict):
                    return
                for k, v in node.items():
                    if k in out and isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0:
                        out[k] = float(v)
                        found += 1
                    elif isinstance(v, dict):
                        look(v)
            look(raw)
            if found:
                return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi in the background while the timed region runs (reading only)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons)}


def weight_bytes(cfg, n_layers) -> int:
    """Bytes of every weight a decode step reads once (bfloat16): the layers' matrices and
    norm vectors, the final norm, and the head (the tied embedding table, read whole by the
    head; the embedding lookup reads one row per sequence, which is not counted)."""
    d, qd = cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim
    kvd, f = cfg.num_key_value_heads * cfg.head_dim, cfg.intermediate_size
    per_layer = (qd + 2 * kvd) * d + d * qd + 2 * f * d + d * f
    norms = 4 * d * 4                       # float32 vectors
    return n_layers * (per_layer * 2 + norms) + d * 4 + cfg.vocab_size * d * 2


def kv_bytes_at(cfg, n_layers, length) -> int:
    """Cache bytes one sequence of `length` tokens makes a decode step read (bfloat16 keys
    and values; even layers see the last sliding_window keys only)."""
    per_tok = 2 * cfg.num_key_value_heads * cfg.head_dim * 2
    sliding = sum(1 for l in range(n_layers) if cfg.layer_is_sliding(l))
    return per_tok * (sliding * min(length, cfg.sliding_window) + (n_layers - sliding) * length)


def prefill_flops(cfg, n_layers, t) -> float:
    d, qd = cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim
    kvd, f = cfg.num_key_value_heads * cfg.head_dim, cfg.intermediate_size
    linear = 2.0 * t * ((qd + 2 * kvd) * d + d * qd + 3 * f * d)
    flops = 0.0
    for l in range(n_layers):
        w = cfg.sliding_window if cfg.layer_is_sliding(l) else t
        pairs = sum(min(p + 1, w) for p in range(t))
        flops += linear + 4.0 * cfg.head_dim * cfg.num_attention_heads * pairs
    return flops + 2.0 * d * cfg.vocab_size          # the head runs on the last row


def fill_cache_random(runner):
    import torch
    for g in runner.cache.groups:
        for t in g.k + g.v:
            flat = t.view(-1)
            for lo in range(0, flat.numel(), 1 << 28):
                flat[lo:lo + (1 << 28)].normal_(0.0, 0.5)


MIXED = (1.0, 0.5, 0.25, 0.125, 0.0625, 0.0625, 0.03125, 0.03125)     # --mixed-lengths: fractions of the context, in turn


def measure_decode(eng, batch, ctx, steps, warmup, rng, clocks=None, mixed=False):
    """K timed decode steps that end at length ctx (with `mixed`: at the fractions MIXED of it, in turn).  Returns
    (device ms per step, e2e ms per step, kernel launches in the timed region, h2d bytes per step, d2h bytes per
    step, mean length, or with `mixed` the list of the sequences' mean lengths)."""
    import torch
    r = eng.runner
    vocab = r.vocab_size
    ends = [max(warmup + steps + 1, int(ctx * MIXED[i % len(MIXED)])) if mixed else ctx for i in range(batch)]
    starts = [e - (warmup + steps) for e in ends]

    def prepare():
        slots = r.admit(batch)
        r.cache.extend_all(slots, starts)
        return slots

    # ---- device-timed: steps issued back to back, tokens stay on the device ----
    slots = prepare()
    toks = [[rng.randrange(vocab)] for _ in range(batch)]
    ms_dev, launches = r.decode_steps_timed(slots, toks, warmup, steps, clocks)
    for s in slots:
        r.release(s)

    # ---- end to end: the public entry point (Engine.generate_from_ids on conversations that hold the
    # context), token ids back on the host; every step uploads which slots run and brings its tokens back ----
    convs = eng.open(batch)
    r.cache.extend_all([c.slot for c in convs], starts)
    r.write_records([c.slot for c in convs], pos=starts)
    for c, start in zip(convs, starts):
        c.position = start
    kw = dict(temp=0.0, top_k=0, top_p=1.0, rep_penalty=1.0, stop_ids=[])
    eng.generate_from_ids(convs, [[rng.randrange(vocab)] for _ in range(batch)], max_tokens=warmup, **kw)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.generate_from_ids(convs, [[] for _ in range(batch)], max_tokens=steps, **kw)
    torch.cuda.synchronize()
    ms_e2e = (time.perf_counter() - t0) * 1e3 / steps
    assert all(len(o) == steps for o in outs), "every sequence decodes every step"
    for c in convs:
        c.close()
    from hos_b200.engine.decode import META, bucket_for
    h2d = (META + bucket_for(batch)) * 4       # live rows, stop ids, the slots that run
    d2h = bucket_for(batch) * 4                # the sampled ids
    mean_len = [e - steps / 2.0 for e in ends] if mixed else ctx - steps / 2.0
    return ms_dev, ms_e2e, launches, h2d, d2h, mean_len


def measure_prefill(eng, tokens, rng, reps=3, pieces=1):
    """Milliseconds of one prompt of `tokens` tokens (the best of `reps` runs after a warm-up
    run), fed whole or as `pieces` steps of equal size that continue one another."""
    import torch
    r = eng.runner
    prompt = [rng.randrange(r.vocab_size) for _ in range(tokens)]
    size = (tokens + pieces - 1) // pieces
    best = None
    for i in range(reps + 1):
        slot = r.admit(1)[0]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for lo in range(0, tokens, size):
            r.step([slot], [prompt[lo:lo + size]])
        e1.record()
        torch.cuda.synchronize()
        r.release(slot)
        ms = e0.elapsed_time(e1)
        if i > 0:                              # the first run warms up
            best = ms if best is None else min(best, ms)
    return best


def run_baseline_workload(args) -> int:
    """The workloads that go with the 9B and 27B layer sizes: 9B, 16 prompts of seeded lengths
    U[64, 2048] in one ragged prompt step, then 256 greedy tokens each, context 4096; 27B, 8 prompts of
    1,024 tokens, then 256 each; 2B, 8 prompts of 512 and decoding as far as --decode-tokens says.
    Method of the reference's own bench (src/lib.rs:683-727): one warm-up prompt step, then the prompt
    step and the greedy decoding timed apart, through `Engine.bench`, the public entry point."""
    import random
    import torch
    from hos_b200 import Engine
    from hos_b200 import models  # noqa: F401
    from hos_b200.registry import config_from_dict
    full_layers = MODELS[args.model]["num_hidden_layers"]
    layers = args.layers or full_layers
    ctx = 4096 if args.model != "2b" else 8192
    cfg = config_from_dict(dict(MODELS[args.model], num_hidden_layers=layers, max_position_embeddings=ctx))
    rng = random.Random(0)
    if args.model == "9b":
        lens = [rng.randint(64, 2048) for _ in range(16)]
    elif args.model == "27b":
        lens = [1024] * 8
    else:
        lens = [512] * 8
    decode = args.decode_tokens
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in lens]
    pk, pk_src = peaks()
    eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_batch=len(lens),
                             max_tokens=sum((n + decode + 63) // 64 * 64 for n in lens), max_seq_len=ctx)
    clocks = ClockSampler(torch.cuda.current_device())
    clocks.start()
    n_prompt, pre_s, pre_tps, produced, dec_s, dec_tps = eng.bench(prompts, decode)
    clock_rec = clocks.stop()
    fl = sum(prefill_flops(cfg, layers, n) for n in lens)
    steps = produced / len(lens)
    wbytes = weight_bytes(cfg, layers)
    step_bytes = wbytes + sum(kv_bytes_at(cfg, layers, n + int(steps / 2)) for n in lens)
    ms_step = dec_s * 1e3 / max(steps, 1e-9)
    print(json.dumps({
        "workload": "baseline", "model": f"gemma-2-{args.model} sizes, random weights", "layers": layers,
        "layers_full": full_layers, "batch": len(lens), "prompt_tokens": n_prompt, "prompt_lengths": "U[64,2048] seeded"
        if args.model == "9b" else str(lens[0]), "context": ctx, "dtype": "bf16", "peaks": pk_src, "clocks": clock_rec,
        "prefill": {"tokens": n_prompt, "ms": pre_s * 1e3, "value": pre_tps, "unit": "tok/s", "tflop": fl / 1e12,
                    "frac": fl / pre_s / (pk["bf16_tflops_sustained"] * 1e12), "peak_tflops": pk["bf16_tflops_sustained"],
                    "of": pk_src + " (sustained)"},
        "decode": {"tokens": produced, "steps": steps, "ms_per_step": ms_step, "value": dec_tps, "unit": "tok/s",
                   "bytes_per_step": step_bytes, "achieved_gbs": step_bytes / (ms_step * 1e-3) / 1e9,
                   "frac": step_bytes / (ms_step * 1e-3) / 1e9 / pk["hbm_gbs"], "peak_gbs": pk["hbm_gbs"], "of": pk_src}}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has, for a quick run")
    ap.add_argument("--model", default="2b", choices=sorted(MODELS), help="layer sizes (default: Gemma-2 2B)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--workload", default="step", choices=["step", "baseline"],
                    help="step: the decode step at the context's end (the default line); baseline: prompts then 256 "
                         "greedy tokens, the workload that goes with the model's sizes")
    ap.add_argument("--decode-tokens", type=int, default=256, help="tokens decoded per sequence by --workload baseline")
    ap.add_argument("--mixed-lengths", action="store_true",
                    help="the sequences end at 1, 1/2, 1/4, 1/8, 1/16, 1/16, 1/32, 1/32 of the context, in turn, "
                         "instead of all at its end (not the driver's line: how a batch of unequal lengths decodes)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="length of the timed prompt (default: the contract's 2,048)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate: no cargo/rustc in this image and no network "
                          "to fetch its 38 crates; it also runs Gemma-2 on the CPU only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this library runs on a single GPU, --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "baseline":
        return run_baseline_workload(args)

    import random
    import torch
    from hos_b200 import Engine
    from hos_b200 import models  # noqa: F401
    from hos_b200.registry import config_from_dict

    full_layers = MODELS[args.model]["num_hidden_layers"]
    if args.layers is None:
        args.layers = full_layers
    raw = dict(MODELS[args.model], num_hidden_layers=args.layers)
    cfg = config_from_dict(raw)
    pk, pk_src = peaks()
    rng = random.Random(0)
    batches = [args.batch] + ([] if args.no_points else [1, 64])
    cap_tokens = max(batches) * ((args.ctx + 63) // 64 * 64)
    eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_batch=max(batches), max_tokens=cap_tokens,
                             max_seq_len=args.ctx)
    fill_cache_random(eng.runner)
    torch.cuda.synchronize()

    clocks = ClockSampler(torch.cuda.current_device())
    ms_dev, ms_e2e, launches, h2d, d2h, mean_len = measure_decode(
        eng, args.batch, args.ctx, args.steps, args.warmup, rng, clocks, mixed=args.mixed_lengths)
    clock_rec = clocks.result

    wbytes = weight_bytes(cfg, args.layers)
    if args.mixed_lengths:
        step_bytes = wbytes + sum(kv_bytes_at(cfg, args.layers, int(n)) for n in mean_len)
    else:
        step_bytes = wbytes + args.batch * kv_bytes_at(cfg, args.layers, int(mean_len))
    achieved = step_bytes / (ms_dev * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Gemma-2 2B)",
        "value": args.batch * 1e3 / ms_dev, "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": f"gemma-2-{args.model} sizes, random weights", "global_batch": args.batch, "seq_len": args.ctx,
            "parallelism": "single_gpu", "layers": args.layers, "layers_full": full_layers,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "sliding_window": cfg.sliding_window,
            "decode_ends_at": "1, 1/2, 1/4, 1/8, 1/16, 1/16, 1/32, 1/32 of %d in turn" % args.ctx if args.mixed_lengths else args.ctx,
            "cache_fill": "random keys and values", "l2": "inputs larger than L2 (weights %.1f GB per step)" % (wbytes / 1e9),
            "peaks": pk_src, "prefill_tokens": args.prefill_tokens},
        "clocks": clock_rec,
        "e2e": {"value": args.batch * 1e3 / ms_e2e, "unit": "tok/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": step_bytes, "of": pk_src},
    }
    if not args.no_prefill:
        ms = measure_prefill(eng, args.prefill_tokens, rng)
        fl = prefill_flops(cfg, args.layers, args.prefill_tokens)
        line["prefill"] = {"value": args.prefill_tokens * 1e3 / ms, "tokens": args.prefill_tokens, "ms": ms,
                           "frac": fl / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), "tflop": fl / 1e12,
                           "peak_tflops": pk["bf16_tflops"], "of": pk_src}
        if args.prefill_tokens % 4 == 0:       # the same prompt as four steps that continue one another
            line["prefill"]["ms_in_4_pieces"] = measure_prefill(eng, args.prefill_tokens, rng, pieces=4)
    if not args.no_points:
        pts, pts_e2e = {}, {f"decode_b{args.batch}": line["e2e"]["value"]}
        for b in (1, 64):
            m, me, _, _, _, _ = measure_decode(eng, b, args.ctx, args.steps, args.warmup, rng)
            pts[f"decode_b{b}"] = b * 1e3 / m
            pts_e2e[f"decode_b{b}"] = b * 1e3 / me
        line["points"] = pts
        line["points_e2e"] = pts_e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
