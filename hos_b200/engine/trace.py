"""Trace replay: feed given token ids through the model step by step and write the
logits.  Nothing is sampled.  It drives the same `Runner.step`, cache and kernels
that generation uses.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries`: each request's next tokens (one or many, from the request's first token
or from where its last step left it) and the places among them whose logits are
wanted.  A request that is seen for the first time gets a slot, whether or not
other requests of the step are under way.
`end`: requests that are finished after this step; their slots and pages go back.
For a step that wants something, DIR/<step>.f32 holds the logits at the wanted
places, in the order of the entries and of `want`, little-endian float32
[wanted, vocab].  After every step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict



def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to 64")
    ap.add_argument("--chunk-tokens", type=int, default=2048,
                    help="most tokens one pass adds to a request that is under way (more are run as several "
                         "passes); layers with a window keep a ring of window + this many keys")
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)

    print("[hos] loading the model (kernels are compiled at their first use)", file=sys.stderr, flush=True)
    from .. import ops
    from .runner import Runner
    # the cache alone bounds a request's length here: replay is not cut at the model's
    # max_position_embeddings, which generation takes as its context limit
    runner = Runner.from_folder(args.model, dtype=args.dtype, max_tokens=args.max_tokens,
                                max_seq_len=args.max_tokens, chunk_tokens=args.chunk_tokens)
    slots: Dict[str, int] = {}

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        step = obj["step"]
        entries = obj.get("entries", [])
        new = [e for e in entries if str(e["id"]) not in slots]
        if new:
            for e, s in zip(new, runner.admit(len(new))):
                slots[str(e["id"])] = s
        if entries:
            logits = runner.step([slots[str(e["id"])] for e in entries],
                                 [e["tokens"] for e in entries],
                                 [e.get("want", []) for e in entries])
            if logits.shape[0] > 0:
                arr = logits.detach().cpu().numpy().astype("<f4", copy=False)
                ops.check_errors()        # the copy waited for the step: a kernel that gave up a wait shows now
                arr.tofile(os.path.join(args.out, f"{step}.f32"))
        for rid in obj.get("end", []):
            runner.release(slots.pop(str(rid)))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
