"""Command line: generate from a model folder.

    python -m mini_sglang_b200.engine.cli --model DIR --input_ids 1,2,3 [--input_ids 4,5] \
        [--prompt "text"] [--prompt_file FILE] [--max_new_tokens 64] [--temperature 0] [--ignore_eos]
        [engine options: --page_size --max_num_reqs --schedule_policy --gpu_memory_utilization
         --random_seed --disable_radix_cache --disable_cuda_graph --max_capture_bs
         --schedule-conservativeness --max_prefill_tokens --dummy_load --dtype --num_pages ...]

Engine options have the names of the reference's launcher (`python -m mini_sglang.launch_server`,
mini_sglang/managers/server_args.py:62-183); the reference starts an HTTP server, this prints one
JSON line per request (token ids, text if the folder has a tokenizer, and the meta information).
"""

from __future__ import annotations

import argparse
import json
import sys

from .args import EngineArgs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mini_sglang_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    EngineArgs.add_cli_args(ap)
    ap.add_argument("--input_ids", action="append", default=[], help="comma-separated token ids (repeatable)")
    ap.add_argument("--prompt", action="append", default=[], help="text prompt (repeatable; needs a tokenizer)")
    ap.add_argument("--prompt_file", type=str, default=None, help="one request per line: JSON list of ids, or text")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--max_new_tokens", type=int, default=64)
    ap.add_argument("--ignore_eos", action="store_true")
    ns = ap.parse_args(argv)
    args = EngineArgs.from_cli_args(ns)

    prompts = [("ids", [int(x) for x in s.replace(" ", "").split(",") if x]) for s in ns.input_ids]
    prompts += [("text", p) for p in ns.prompt]
    if ns.prompt_file:
        with open(ns.prompt_file) as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                prompts.append(("ids", json.loads(line)) if line.startswith("[") else ("text", line))
    if not prompts:
        ap.error("give at least one of --input_ids, --prompt, --prompt_file")

    from .engine import Engine

    engine = Engine(args)
    sp = {"temperature": ns.temperature, "max_new_tokens": ns.max_new_tokens, "ignore_eos": ns.ignore_eos}
    reqs = [engine.add_request(prompt=p if kind == "text" else None, sampling_params=sp,
                               input_ids=p if kind == "ids" else None) for kind, p in prompts]
    import time
    t0 = time.time()
    engine._run_until(reqs)
    for r in reqs:
        print(json.dumps(engine._result(r, t0)), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
