"""Trace replay: feed given token ids through the model step by step and write logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--page-size P]

Reads one JSON object per line from standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch for the engine's step function (the same model, cache
manager and kernels that generation uses; nothing is sampled).  For a step in which logits are
wanted, `<out>/<step>.f32` holds them as little-endian float32 [wanted, vocab], in the order of
the entries and of `want`.  After every step a line `done <step>` is printed and flushed.
Requests named in `end` give back what they hold after the step.  The cache pool is sized for
`--max-tokens` tokens held by live requests, each request rounded up to a multiple of 64, so
pages are used again.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page; must divide 64")
    ap.add_argument("--max-requests", type=int, default=8, help="request slots (live requests at a time)")
    ap.add_argument("--no-cuda-graph", action="store_true")
    args = ap.parse_args(argv)
    if args.page_size < 1 or 64 % args.page_size:
        ap.error("--page-size must divide 64")
    os.makedirs(args.out, exist_ok=True)

    import torch

    from .step import ModelRunner, StepEntry

    num_pages = max(-(-args.max_tokens // 64) * 64 // args.page_size, 1)
    runner = ModelRunner.from_model_dir(args.model, dtype=args.dtype, page_size=args.page_size, num_pages=num_pages,
                                        max_reqs=args.max_requests, use_cuda_graph=not args.no_cuda_graph)
    slots = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = runner.open()
            entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", [])))
        logits = runner.step(entries)
        if logits.shape[0] > 0:
            arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
            tmp = os.path.join(args.out, f".{step}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        else:
            torch.cuda.synchronize()
        for rid in rec.get("end", []):
            if rid in slots:
                runner.close(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
