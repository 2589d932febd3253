"""Benchmark of the engine's decode step (headline) and prefill on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

Default run: Qwen3-8B layer sizes with random weights (N(0, 0.02), bfloat16), a batch of 8
requests at a context of 4,096 tokens, KV page size 16.  A "step" is one decode step of the
whole batch.  Prints ONE JSON line:

  value      decoded tokens per second, timed on the device (CUDA events around K steps that feed
             given tokens: graph replay + the step's host-to-device staging copy)
  e2e        the same through the Python entry point (Engine.step(): scheduler, pinned staging
             copy, graph replay, sampling kernel, device-to-host read of the sampled ids)
  prefill    one 2,048-token prompt in one step: tokens/s, ms, and flops / time / bf16 peak
  roofline   bytes the decode step has to read (every weight once + the live requests' cache)
             divided by its time, against the measured copy bandwidth
  points     decode tokens/s at batch 1 and 64

Peaks come from MEASURED_PEAKS.json beside this file when present.  Every timed step reads far
more than the 126 MB L2 (15 GB of weights), so L2 is not flushed between iterations.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 36, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 40960, "hidden_act": "silu", "attention_bias": False, "torch_dtype": "bfloat16",
    "eos_token_id": 151645,
}
FULL_LAYERS = 36
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self):
        return len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, lo=0, hi=None):
        rows = [r for r in self.rows[lo:hi] if len(r) >= 6 and r[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        sm = sorted(int(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def _unavailable(why):
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def reference_arm(args):
    """The unmodified reference (installed under baseline/_ref) through its own public API:
    Engine(ServerArgs(...)).async_generate with token ids.  Decode tokens/s = B * (N2 - N1) / (T(N2) - T(N1)) for
    two runs of B concurrent requests that differ only in max_new_tokens; prefill = a 2,048-token request with
    one new token.  Its attention comes from the flash_attn 2.x wheel (backend fa2, page size 256: the only one
    of its backends that has its wheel on this box; fa3 needs sgl_kernel and refuses sm_100)."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "mini_sglang")):
        return _unavailable("reference not installed under baseline/_ref")
    import asyncio
    import multiprocessing
    import signal

    W, K, B, CTX, PREFILL = max(args.warmup, 3), args.steps, args.batch, args.context, 2048
    tmp = tempfile.mkdtemp(prefix="msgl_ref_")
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(QWEN3_8B, f)
    try:
        from tokenizers import Tokenizer, models, pre_tokenizers
        tok = Tokenizer(models.WordLevel({f"t{i}": i for i in range(QWEN3_8B["vocab_size"])}, unk_token="t0"))
        tok.pre_tokenizer = pre_tokenizers.Whitespace()
        tok.save(os.path.join(tmp, "tokenizer.json"))
        with open(os.path.join(tmp, "tokenizer_config.json"), "w") as f:
            json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "t0"}, f)
    except Exception as e:                                    # noqa: BLE001
        return _unavailable(f"could not write a stand-in tokenizer for the reference's front end: {e}")

    def cleanup():
        for ch in multiprocessing.active_children():
            ch.terminate()

    def on_alarm(signum, frame):
        cleanup()
        _unavailable("the reference did not finish within its time limit on this box")
        os._exit(0)

    signal.signal(signal.SIGALRM, on_alarm)
    signal.alarm(1500)
    sys.path.insert(0, ref)
    try:
        import torch
        from mini_sglang import Engine, ServerArgs
        engine = Engine(ServerArgs(model=tmp, attention_backend="fa2", page_size=256, dummy_load=True,
                                   max_prefill_tokens=1 << 20, gpu_memory_utilization=0.6, random_seed=0, disable_cuda_graph=True,
                                   log_level="ERROR"))
        gen = torch.Generator().manual_seed(0)
        V = QWEN3_8B["vocab_size"]
        loop = asyncio.new_event_loop()          # the caller owns the loop the reference's front end runs on
        asyncio.set_event_loop(loop)

        def run(n_req, prompt_len, max_new):
            prompts = [torch.randint(0, V, (prompt_len,), generator=gen).tolist() for _ in range(n_req)]
            sp = {"temperature": 0.0, "max_new_tokens": max_new, "ignore_eos": True}

            async def go():
                t0 = time.perf_counter()
                outs = await asyncio.gather(*[engine.async_generate(input_ids=p, sampling_params=sp) for p in prompts])
                return time.perf_counter() - t0, outs
            dt, outs = loop.run_until_complete(go())
            assert all(o["meta_info"]["completion_tokens"] == max_new for o in outs)
            return dt

        n1, n2 = W, W + K
        prompt_len = CTX - n2 - 1
        run(B, prompt_len, n1)                                  # warm-up
        t1 = min(run(B, prompt_len, n1) for _ in range(2))
        t2 = min(run(B, prompt_len, n2) for _ in range(2))
        ms_step = (t2 - t1) / K * 1e3
        value = B / (ms_step * 1e-3)
        run(1, PREFILL, 1)
        pf = min(run(1, PREFILL, 1) for _ in range(3))
        line = {"metric": "decode tokens/s, Qwen3-8B shape, batch 8, context 4096 (one B200)", "value": round(value, 1),
                "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic: random weights (the reference's dummy_load), uniform random token ids",
                "config": {"model": "Qwen3-8B shape", "layers": 36, "global_batch": B, "seq_len": CTX, "page_size": 256,
                           "attention_backend": "fa2", "cuda_graph": False, "timing": "wall clock through Engine.async_generate, difference of two runs"},
                "e2e": {"value": round(value, 1), "unit": "tokens/s"},
                "prefill": {"value": round(PREFILL / pf, 1), "tokens": PREFILL, "ms": round(pf * 1e3, 3)},
                "impl": "reference"}
        print(json.dumps(line))
    except BaseException as e:                                   # noqa: BLE001
        _unavailable(f"the reference failed on this box: {type(e).__name__}: {str(e)[:300]}")
    finally:
        signal.alarm(0)
        cleanup()
    sys.stdout.flush()
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="decode / prefill: run that timed region alone and print a short line (for profilers)")
    ap.add_argument("--profiler-range", action="store_true",
                    help="cudaProfilerStart/Stop around the timed region (ncu --profile-from-start off)")
    ap.add_argument("--no-graph", action="store_true", help="decode without CUDA graphs")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures the single-GPU engine; --gpus {args.gpus} is not supported (this engine has no multi-GPU path)")
        return 2
    if args.impl == "reference":
        return reference_arm(args)

    import torch

    from mini_sglang_b200 import Engine, EngineArgs, ops
    from mini_sglang_b200.engine.step import StepEntry

    W, K = max(args.warmup, 3), args.steps
    B, CTX, PAGE, PREFILL = args.batch, args.context, 16, 2048
    cfg = dict(QWEN3_8B)
    cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    tmp = tempfile.mkdtemp(prefix="msgl_bench_")
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(cfg, f)
    if args.only != "all":
        args.skip_points = True
    max_b = B if args.skip_points else max(B, 64)
    pages = max_b * (CTX // PAGE + 2) + 256
    eng = Engine(EngineArgs(model=tmp, dummy_load=True, random_seed=0, page_size=PAGE, num_pages=pages,
                            max_num_reqs=max_b + 2, max_context_len=CTX + 64, max_prefill_tokens=8192, chunk_size=2048,
                            disable_radix_cache=True, schedule_policy="fcfs", log_level="WARNING",
                            disable_cuda_graph=args.no_graph))
    runner = eng.runner
    V, H, L = cfg["vocab_size"], cfg["hidden_size"], cfg["num_hidden_layers"]
    nq, nkv, d, I = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"]
    gen = torch.Generator().manual_seed(0)

    def rand_tokens(n):
        return torch.randint(0, V, (n,), generator=gen).tolist()

    layer_params = H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I + 2 * H + 2 * d
    weight_bytes = 2 * (L * layer_params + V * H + H)            # every weight a decode step reads once (head included)
    kv_bytes_per_token = L * 2 * nkv * d * 2

    clocks = ClockSampler()
    clocks.start()

    def timed_decode(batch, steps, warm):
        """Feed given tokens: `batch` requests at context CTX - (warm + steps) .. CTX."""
        prompt_len = CTX - (warm + steps) - 1
        slots = [runner.open() for _ in range(batch)]
        for s in slots:                                           # prompts in portions of 2,048
            toks = rand_tokens(prompt_len)
            for i in range(0, prompt_len, 2048):
                runner.step([StepEntry(s, toks[i:i + 2048], [])])
        feed = [[rand_tokens(1) for _ in slots] for _ in range(warm + steps)]
        for i in range(warm):
            runner.step([StepEntry(s, t, [0]) for s, t in zip(slots, feed[i])])
        torch.cuda.synchronize()
        l0 = ops.LAUNCHES
        c0 = clocks.mark()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if args.profiler_range:
            torch.cuda.profiler.start()
        e0.record()
        for i in range(warm, warm + steps):
            runner.step([StepEntry(s, t, [0]) for s, t in zip(slots, feed[i])])
        e1.record()
        torch.cuda.synchronize()
        if args.profiler_range:
            torch.cuda.profiler.stop()
        ms = e0.elapsed_time(e1) / steps
        launches = ops.LAUNCHES - l0
        c1 = clocks.mark()
        for s in slots:
            runner.close(s)
        return ms, launches, (c0, c1)

    if args.only == "prefill":
        s = runner.open()
        toks = rand_tokens(PREFILL)
        for i in range(W):
            s2 = runner.open()
            runner.step([StepEntry(s2, toks, [PREFILL - 1])])
            runner.close(s2)
        torch.cuda.synchronize()
        if args.profiler_range:
            torch.cuda.profiler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry(s, toks, [PREFILL - 1])])
        e1.record()
        torch.cuda.synchronize()
        if args.profiler_range:
            torch.cuda.profiler.stop()
        clocks.stop()
        print(json.dumps({"only": "prefill", "layers": L, "tokens": PREFILL, "ms": round(e0.elapsed_time(e1), 3)}))
        return 0

    # ---- headline: decode at batch B, device-timed
    ms_step, launches, (c0, c1) = timed_decode(B, K, W)
    if args.only == "decode":
        clocks.stop()
        print(json.dumps({"only": "decode", "layers": L, "batch": B, "context": CTX, "ms_per_step": round(ms_step, 4),
                          "launches": launches}))
        return 0
    value = B / (ms_step * 1e-3)
    step_bytes = weight_bytes + B * (CTX - K // 2) * kv_bytes_per_token
    achieved = step_bytes / (ms_step * 1e-3) / 1e9

    # ---- end to end through the Python entry point: host tokens in, host tokens out
    # Prompts are prefilled in portions, so the requests get their first token a few steps apart; max_new_tokens
    # leaves room for that, so that none of them finishes inside the timed steps.
    prompt_len = CTX - (W + K) - 16
    reqs = [eng.add_request(input_ids=rand_tokens(prompt_len),
                            sampling_params={"temperature": 0.0, "max_new_tokens": W + K + 15, "ignore_eos": True})
            for _ in range(B)]
    while any(len(r.output) == 0 for r in reqs):
        eng.step()
    for _ in range(W - 1):
        eng.step()
    torch.cuda.synchronize()
    done0 = sum(len(r.output) for r in reqs)
    t0 = time.perf_counter()
    for _ in range(K):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    done = sum(len(r.output) for r in reqs) - done0
    assert done == B * K, "a request finished inside the timed steps"
    while not eng.scheduler.idle:
        eng.step()
    key = next(iter(runner._graphs)) if runner._graphs else None
    h2d = 4 * max((g.layout.size for g in runner._graphs.values() if g.layout.B == runner._bucket(B)), default=0)
    e2e = {"value": round(done / dt, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B}

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            ms_b, _, _ = timed_decode(b, max(K // 2, 8), W)
            points[f"decode_b{b}"] = round(b / (ms_b * 1e-3), 1)

    # ---- prefill of 2,048 tokens in one step
    pf_ms = []
    for i in range(3 + 5):
        s = runner.open()
        toks = rand_tokens(PREFILL)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry(s, toks, [PREFILL - 1])])
        e1.record()
        torch.cuda.synchronize()
        if i >= 3:
            pf_ms.append(e0.elapsed_time(e1))
        runner.close(s)
    pf = sorted(pf_ms)[len(pf_ms) // 2]
    lin_flops = 2 * PREFILL * L * (layer_params - 2 * H - 2 * d) + 2 * V * H
    attn_flops = L * 4 * nq * d * PREFILL * (PREFILL + 1) // 2
    pf_flops = lin_flops + attn_flops
    prefill = {"value": round(PREFILL / (pf * 1e-3), 1), "tokens": PREFILL, "ms": round(pf, 3),
               "frac": round(pf_flops / (pf * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    clocks.stop()
    line = {
        "metric": "decode tokens/s, Qwen3-8B shape, batch 8, context 4096 (one B200)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": {"model": "Qwen3-8B shape", "layers": L, "layers_full": FULL_LAYERS, "hidden": H, "q_heads": nq,
                   "kv_heads": nkv, "head_dim": d, "intermediate": I, "vocab": V, "global_batch": B, "seq_len": CTX,
                   "page_size": PAGE, "prefill_tokens": PREFILL, "parallelism": "single GPU", "cuda_graph": True,
                   "l2": "inputs larger than L2 (15 GB of weights per step), no flush", "peaks": pk["source"]},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks.summary(c0, c1), "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
