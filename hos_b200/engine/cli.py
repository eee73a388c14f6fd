"""The command line, in the manner of the reference's `hos` (src/main.rs:3459-3577, :3248-3295,
:65-101): the same option names and defaults where it has them.

    hos -m <dir> -p <ids> [-n 64] [--temp 0.0] [--top-k 40] [--top-p 0.95]
        [--repeat-penalty 1.1] [--repeat-last-n 64] [--seed 42] [--no-echo]
    hos -m <dir> --bench [-n 64] [-p <ids>] [--batch B] [--prompt-len T] [--ctx C]   # prompt and decode throughput
    hos -m <dir> --perplexity <ids>                # score a token sequence

Prompts are token ids separated by commas (tokenizers are not part of this library); -p may
be given several times, which makes a batch.  The model is `-m`, else $HOS_MODEL
(src/main.rs:3419-3425).  `--fp32` runs everything in true 32-bit; `--random <config.json>`
runs that configuration with random weights from `--seed` instead of a model folder.
stdout carries token ids only; everything else goes to stderr with the reference's `[hos]`
prefix.  An unknown option ends with status 2 (src/main.rs:3547-3554).
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import List, Optional

USAGE = """usage: hos -m model_dir -p "id,id,..." [-n 64] [--temp 0.0] [--seed 42]
       hos -m model_dir --bench                  # prefill/decode throughput
       hos -m model_dir --perplexity "id,id,..." # score a token sequence
options: --top-k 40 --top-p 0.95 --repeat-penalty 1.1 --repeat-last-n 64 --no-echo --fp32
         --random config.json (random weights from --seed instead of -m)
         --ctx C (longest sequence the cache is sized for)
         --bench: --batch B sequences of --prompt-len T fixed ids each (default: one prompt of 16)"""


def parse_ids(text: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(" ", "").split(",") if t != ""]
    except ValueError:
        print(f"[hos] a prompt is token ids separated by commas, found {text!r}", file=sys.stderr)
        sys.exit(2)


class Args:
    def __init__(self):
        self.model: Optional[str] = None
        self.prompts: List[List[int]] = []
        self.n_predict, self.temp, self.top_k, self.top_p = 64, 0.0, 40, 0.95
        self.rep_penalty, self.repeat_last_n, self.seed = 1.1, 64, 42
        self.gpu, self.no_echo, self.bench, self.fp32 = True, False, False, False
        self.perplexity: Optional[List[int]] = None
        self.random: Optional[str] = None
        self.batch, self.prompt_len, self.ctx = 1, 16, None


def parse_args(argv: List[str]) -> Args:
    a = Args()
    it = iter(argv)

    def value(flag: str) -> str:
        try:
            return next(it)
        except StopIteration:
            print(f"[hos] a value is expected after {flag}", file=sys.stderr)
            sys.exit(2)
    for arg in it:
        if arg in ("-m", "--model"):
            a.model = value(arg)
        elif arg in ("-p", "--prompt"):
            a.prompts.append(parse_ids(value(arg)))
        elif arg in ("-n", "--n-predict"):
            a.n_predict = int(value(arg))
        elif arg == "--temp":
            a.temp = float(value(arg))
        elif arg == "--top-k":
            a.top_k = int(value(arg))
        elif arg == "--top-p":
            a.top_p = float(value(arg))
        elif arg == "--repeat-penalty":
            a.rep_penalty = float(value(arg))
        elif arg == "--repeat-last-n":
            a.repeat_last_n = int(value(arg))
        elif arg == "--seed":
            a.seed = int(value(arg))
        elif arg == "--gpu":
            a.gpu = True
        elif arg == "--no-echo":
            a.no_echo = True
        elif arg == "--bench":
            a.bench = True
        elif arg == "--fp32":
            a.fp32 = True
        elif arg == "--random":
            a.random = value(arg)
        elif arg == "--perplexity":
            a.perplexity = parse_ids(value(arg))
        elif arg == "--batch":
            a.batch = max(1, int(value(arg)))
        elif arg == "--prompt-len":
            a.prompt_len = max(1, int(value(arg)))
        elif arg == "--ctx":
            a.ctx = max(1, int(value(arg)))
        elif arg in ("-h", "--help"):
            print(USAGE, file=sys.stderr)
            sys.exit(0)
        else:
            print(f"[hos] unknown argument: {arg}", file=sys.stderr)
            print("[hos] (note: don't type the [ ] brackets from docs — they mean 'optional')", file=sys.stderr)
            print("[hos] run `hos --help` for usage", file=sys.stderr)
            sys.exit(2)
    return a


def bench_prompt(vocab: int, length: int = 16, which: int = 0) -> List[int]:
    """A fixed prompt, so that numbers compare from run to run (the reference's is a fixed
    sentence, src/main.rs:44; here fixed ids, another run of them for each sequence of a batch)."""
    return [((i + 1000003 * which) * 7919 + 13) % vocab for i in range(1, length + 1)]


def main(argv: Optional[List[str]] = None) -> int:
    print("[hos] hos_b200: Gemma-2 generation on one B200", file=sys.stderr)
    args = parse_args(list(sys.argv[1:] if argv is None else argv))
    t0 = time.perf_counter()
    if not args.random and not (args.model or os.environ.get("HOS_MODEL")):
        print("[hos] no model: give -m <dir> or set HOS_MODEL", file=sys.stderr)
        return 1
    from .. import HosError
    from .engine import Engine
    dtype = "float32" if args.fp32 else "bfloat16"
    n_seqs = max(1, len(args.prompts), args.batch if args.bench else 1)
    size = {}
    if args.ctx is not None:
        size = dict(max_seq_len=args.ctx, max_tokens=n_seqs * ((args.ctx + 63) // 64 * 64))
    try:
        if args.random:
            from .. import models  # noqa: F401
            from ..registry import config_from_dict
            with open(args.random) as f:
                cfg = config_from_dict(json.load(f))
            eng = Engine.from_config(cfg, seed=args.seed, dtype=dtype, max_batch=n_seqs, **size)
        else:
            model = args.model or os.environ.get("HOS_MODEL")
            eng = Engine(model, gpu=args.gpu, dtype=dtype, max_batch=n_seqs, **size)
    except (HosError, OSError) as e:
        print(f"[hos] error: {e}", file=sys.stderr)
        return 1
    print(f"[hos] load took {time.perf_counter() - t0:.2f}s", file=sys.stderr)

    if args.bench:
        prompts = args.prompts or [bench_prompt(eng.vocab_size(), args.prompt_len, i) for i in range(args.batch)]
        try:
            b = eng.bench(prompts if len(prompts) > 1 else prompts[0], args.n_predict if args.n_predict > 0 else 64)
        except HosError as e:
            print(f"[hos] error: {e}", file=sys.stderr)
            return 1
        print("=== HOS benchmark ===")
        print(f"backend    : B200 GPU ({dtype})")
        print(f"prefill    : {b[0]} tok in {b[1]:.3f}s  ({b[2]:.1f} tok/s)")
        print(f"decode     : {b[3]} tok in {b[4]:.3f}s  ({b[5]:.1f} tok/s)")
        return 0
    if args.perplexity is not None:
        n, mean, ppl = eng.perplexity(args.perplexity)
        print(f"tokens scored : {n}")
        print(f"mean nll      : {mean:.6f} nats")
        print(f"perplexity    : {ppl:.4f}")
        return 0

    prompts = args.prompts or [list(eng.config.bos_token_id) or [2]]
    print(f"[hos] prompt -> {sum(len(p) for p in prompts)} tokens", file=sys.stderr)
    kw = dict(max_tokens=args.n_predict, temp=args.temp, top_k=args.top_k, top_p=args.top_p,
              rep_penalty=args.rep_penalty, repeat_last_n=args.repeat_last_n, seed=args.seed)
    try:
        if len(prompts) == 1:
            first = [True]
            if not args.no_echo:
                sys.stdout.write(",".join(str(t) for t in prompts[0]))
                sys.stdout.flush()
                first[0] = False

            def emit(_, tok):
                sys.stdout.write(("" if first[0] else ",") + str(tok))
                sys.stdout.flush()
                first[0] = False
            out = eng.generate(prompts[0], on_token=emit, **kw)
            print()
            n = len(out)
        else:
            outs = eng.generate(prompts, **kw)
            for p, o in zip(prompts, outs):
                print(",".join(str(t) for t in (([] if args.no_echo else p) + o)))
            n = sum(len(o) for o in outs)
    except HosError as e:
        print(f"\n[hos] error: {e}", file=sys.stderr)
        return 1
    print(f"[hos] generated {n} tokens", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
