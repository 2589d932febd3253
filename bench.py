"""Benchmark of the engine's decode step (headline) and prefill on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]
    python bench.py --workload qwen3_0.6b_mixed     128 prompts of 64..1,024 tokens, half of them sharing a 256-token
                                                    prefix, 256 new tokens each, through the scheduler (Qwen3-0.6B sizes)
    python bench.py --workload qwen3_32b_long       an 8,192-token prompt in portions of 2,048, then decode at batch 16
                                                    and context 8,192 (Qwen3-32B sizes)
    python bench.py --workload sweep                decode at batch 1 / 8 / 64 and contexts of 1k to 32k, prefill of 512 to
                                                    16,384 tokens, each with its fraction of the measured peak (Qwen3-8B sizes)

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
  points     decode tokens/s at batch 1 and 64 at this context, and at batch 1, 8 and 64 right after
             2,048-token prompts (context 2,048 + the steps run)
  sanity     before anything is timed: a one-layer model of the same widths decodes a token through the same
             CUDA-graph path and its logits are compared with the plain implementation under tests/

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
QWEN3_0_6B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
                  head_dim=128, intermediate_size=3072, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8,
                 head_dim=128, intermediate_size=25600, tie_word_embeddings=False)
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


def model_sizes(cfg):
    """(parameters of one layer, bytes of all weights a decode step reads, cache bytes per token) in bfloat16."""
    V, H, L = cfg["vocab_size"], cfg["hidden_size"], cfg["num_hidden_layers"]
    nq, nkv, d, I = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"]
    layer_params = H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I + 2 * H + 2 * d
    weight_bytes = 2 * (L * layer_params + V * H + H)            # every weight a decode step reads once (head included;
    return layer_params, weight_bytes, L * 2 * nkv * d * 2       # the embedding rows it gathers are a few KB)


def step_flops(cfg, q_lens, kv_lens, wanted):
    """Multiply-adds x 2 of one step: every projection for every token, causal attention, the head on `wanted` rows."""
    V, H, L = cfg["vocab_size"], cfg["hidden_size"], cfg["num_hidden_layers"]
    nq, d = cfg["num_attention_heads"], cfg["head_dim"]
    layer_params, _, _ = model_sizes(cfg)
    T = sum(q_lens)
    lin = 2 * T * L * (layer_params - 2 * H - 2 * d) + 2 * wanted * V * H
    attn = sum(L * 4 * nq * d * (q * (kv - q) + q * (q + 1) // 2) for q, kv in zip(q_lens, kv_lens))
    return lin + attn


def sanity_check(cfg, page):
    """One layer of the benchmark's widths, random weights: a 300-token prompt, then three tokens decoded through
    the CUDA-graph path; the last row's logits against the plain implementation (float32, on the GPU)."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_qwen3
    from mini_sglang_b200.config import Qwen3Config
    from mini_sglang_b200.config.qwen3 import build_qwen3_spec
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    from mini_sglang_b200.parts import expected_tensors
    from mini_sglang_b200.weights import RandomSource
    one = dict(cfg, num_hidden_layers=1, max_position_embeddings=1024)
    spec = build_qwen3_spec(Qwen3Config.from_dict(one))
    src = RandomSource(expected_tensors(spec), 5, torch.bfloat16, "cuda")
    weights = {n: src.draw(n) for n in expected_tensors(spec) if src.has(n)}
    toks = torch.randint(0, one["vocab_size"], (303,), generator=torch.Generator().manual_seed(5)).tolist()
    runner = ModelRunner.from_random(spec, 5, dtype="bfloat16", page_size=page, num_pages=64, max_reqs=2)
    s = runner.open()
    runner.step([StepEntry(s, toks[:300], [])])
    for i in range(300, 303):
        row = runner.step([StepEntry(s, [toks[i]], [0])])[0].float().cpu()
    used_graph = runner.last_step_used_graph
    runner.close(s)
    allow = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    with torch.no_grad():
        want = plain_qwen3.forward_sequence(one, weights, toks, device="cuda", rows=[302])[0].cpu()
    torch.backends.cuda.matmul.allow_tf32 = allow
    err = row - want
    scale = want.pow(2).mean().sqrt().item()
    out = {"layers": 1, "rms_err_frac": round(err.pow(2).mean().sqrt().item() / scale, 5),
           "max_err_frac": round(err.abs().max().item() / scale, 5),
           "argmax_equal": bool(int(row.argmax()) == int(want.argmax())), "cuda_graph": bool(used_graph)}
    del runner, weights, src
    torch.cuda.empty_cache()
    if not (out["rms_err_frac"] < 0.015 and out["max_err_frac"] < 0.09 and used_graph):
        raise SystemExit(f"bench.py: the engine's logits do not match the plain implementation: {out}")
    return out


def parse_lengths(spec, batch):
    """'lo:hi' -> `batch` lengths spread evenly from lo to hi; 'a,bxN,c' -> the list itself (x: repeated)."""
    if ":" in spec:
        lo, hi = (int(x) for x in spec.split(":"))
        return [lo + (hi - lo) * i // max(batch - 1, 1) for i in range(batch)]
    out = []
    for part in spec.split(","):
        n, _, rep = part.partition("x")
        out += [int(n)] * (int(rep) if rep else 1)
    return out


def profile_kernels(step, n_steps, captures=lambda: 0):
    """-> {kernel name: [launches a step, mean microseconds]} of the twelve kernels that `n_steps` calls of step() spend the
    most time in, from the CUDA profiler's trace (kernels inside a replayed graph included).  `captures()` counts the CUDA
    graphs made so far: a trace during which one was captured (its warm-up runs are in it) is taken again."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    for _ in range(4):
        before = captures()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(n_steps):
                step()
            torch.cuda.synchronize()
        if captures() == before:
            break
    acc = {}
    for e in prof.events():
        if e.device_type == torch.autograd.DeviceType.CUDA:
            name = e.name.split("(")[0][:60]
            a = acc.setdefault(name, [0, 0.0])
            a[0] += 1
            a[1] += e.time_range.end - e.time_range.start
    top = sorted(acc.items(), key=lambda kv: -kv[1][1])[:12]
    return {k: [round(v[0] / n_steps, 1), round(v[1] / v[0], 1)] for k, v in top}


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


def _write_config(cfg):
    tmp = tempfile.mkdtemp(prefix="msgl_bench_")
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(cfg, f)
    return tmp


def workload_mixed(args):
    """Qwen3-0.6B sizes through the scheduler: 128 prompts with lengths uniform in 64..1,024, every other one opening
    with the same 256 tokens, 256 new tokens each, all handed to the engine at once (prefix cache on, default policy).
    value = generated tokens / wall time of Engine.generate.  roofline: the bytes the run has to read (the weights once
    per step that the scheduler made, and for every decoded token the cache of its request) / its time, against the
    measured copy bandwidth; the prompts' matrix products are left out of that bound, so it flatters no one."""
    import random

    import torch

    from mini_sglang_b200 import Engine, EngineArgs, ops
    cfg = dict(QWEN3_0_6B)
    pk = peaks()
    N, NEW, SHARED = 128, 256, 256
    rnd = random.Random(0)
    V = cfg["vocab_size"]
    common = [rnd.randrange(V) for _ in range(SHARED)]
    prompts = []
    for i in range(N):
        n = rnd.randint(64, 1024)
        prompts.append(common + [rnd.randrange(V) for _ in range(max(n - SHARED, 8))] if i % 2 == 0
                       else [rnd.randrange(V) for _ in range(n)])
    clocks = ClockSampler()
    clocks.start()
    eng = Engine(EngineArgs(model=_write_config(cfg), dummy_load=True, random_seed=0, page_size=16, max_num_reqs=256,
                            max_context_len=2048, gpu_memory_utilization=0.5, log_level="WARNING"))
    sp = {"temperature": 0.0, "max_new_tokens": NEW, "ignore_eos": True}
    warm = [[rnd.randrange(V) for _ in range(rnd.randint(64, 1024))] for _ in range(N)]
    eng.generate(input_ids=warm, sampling_params=sp)                  # graphs captured, buffers sized
    eng.flush_cache()
    stats0 = dict(eng.scheduler.stats)
    l0, c0 = ops.LAUNCHES, clocks.mark()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.generate(input_ids=prompts, sampling_params=sp)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    c1 = clocks.mark()
    clocks.stop()
    st = {k: v - stats0.get(k, 0) for k, v in eng.scheduler.stats.items()}
    generated = sum(len(o["token_ids"]) for o in outs)
    assert generated == N * NEW
    _, weight_bytes, kv_tok = model_sizes(cfg)
    kv_read = sum(NEW * len(p) + NEW * (NEW - 1) // 2 for p in prompts) * kv_tok
    need = st["steps"] * weight_bytes + kv_read
    achieved = need / dt / 1e9
    eng.scheduler.check_idle_invariants()
    print(json.dumps({
        "workload": "qwen3_0.6b_mixed", "metric": "generated tokens/s through the scheduler, Qwen3-0.6B shape (one B200)",
        "value": round(generated / dt, 1), "unit": "tokens/s", "seconds": round(dt, 3), "dtype": "bf16",
        "data": "synthetic: random weights, uniform random token ids",
        "config": {"model": "Qwen3-0.6B shape", "layers": cfg["num_hidden_layers"], "requests": N, "prompt_tokens": sum(map(len, prompts)),
                   "shared_prefix": SHARED, "new_tokens": NEW, "page_size": 16, "policy": "lpm", "radix_cache": True},
        "scheduler": {"steps": st["steps"], "prefill_tokens": st["prefill_tokens"], "cached_tokens": st["cached_tokens"],
                      "decode_tokens": st["decode_tokens"], "retractions": st["retractions"], "evicted_pages": st["evicted_pages"]},
        "gpu_launches": ops.LAUNCHES - l0, "clocks": clocks.summary(c0, c1),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
        "impl": "ours"}))
    return 0


def workload_long(args):
    """Qwen3-32B sizes (about 65 GB of bfloat16 weights): one 8,192-token prompt fed in portions of 2,048 tokens, timed
    as a whole (flops / time against the measured bf16 peak), then 16 requests decoding at a context of 8,192
    (bytes / time against the measured copy bandwidth)."""
    import torch

    from mini_sglang_b200 import Engine, EngineArgs, ops
    from mini_sglang_b200.engine.step import StepEntry
    cfg = dict(QWEN3_32B)
    cfg["num_hidden_layers"] = args.layers if args.layers != FULL_LAYERS else cfg["num_hidden_layers"]
    pk = peaks()
    W, K = max(args.warmup, 3), min(args.steps, 64)
    B, CTX, PAGE, PORTION = 16, 8192, 16, 2048
    V = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(0)

    def rand_tokens(n):
        return torch.randint(0, V, (n,), generator=gen).tolist()

    clocks = ClockSampler()
    clocks.start()
    eng = Engine(EngineArgs(model=_write_config(cfg), dummy_load=True, random_seed=0, page_size=PAGE,
                            num_pages=(B + 1) * (CTX // PAGE + 2) + 64, max_num_reqs=B + 2, max_context_len=CTX + 64,
                            max_prefill_tokens=8192, chunk_size=PORTION, disable_radix_cache=True, schedule_policy="fcfs",
                            log_level="WARNING"))
    runner = eng.runner
    _, weight_bytes, kv_tok = model_sizes(cfg)

    # ---- the long prompt, portion by portion
    times = []
    for rep in range(3):
        toks = rand_tokens(CTX)
        s = runner.open()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(0, CTX, PORTION):
            runner.step([StepEntry(s, toks[i:i + PORTION], [PORTION - 1] if i + PORTION >= CTX else [])])
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        runner.close(s)
    pf_ms = min(times[1:])
    pf_flops = sum(step_flops(cfg, [PORTION], [i + PORTION], 1 if i + PORTION >= CTX else 0) for i in range(0, CTX, PORTION))

    # ---- decode at batch 16, contexts CTX - (W + K) .. CTX
    prompt_len = CTX - (W + K) - 1
    slots = [runner.open() for _ in range(B)]
    for s in slots:
        toks = rand_tokens(prompt_len)
        for i in range(0, prompt_len, PORTION):
            runner.step([StepEntry(s, toks[i:i + PORTION], [])])
    feed = [[rand_tokens(1) for _ in slots] for _ in range(W + K)]
    for i in range(W):
        runner.step([StepEntry(s, t, [0]) for s, t in zip(slots, feed[i])])
    torch.cuda.synchronize()
    l0, c0 = ops.LAUNCHES, clocks.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(W, W + K):
        runner.step([StepEntry(s, t, [0]) for s, t in zip(slots, feed[i])])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / K
    launches, c1 = ops.LAUNCHES - l0, clocks.mark()
    clocks.stop()
    for s in slots:
        runner.close(s)
    step_bytes = weight_bytes + B * (CTX - K // 2) * kv_tok
    achieved = step_bytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "workload": "qwen3_32b_long", "metric": "decode tokens/s, Qwen3-32B shape, batch 16, context 8192 (one B200)",
        "value": round(B / (ms * 1e-3), 1), "unit": "tokens/s", "steps": K, "warmup": W, "ms_per_step": round(ms, 4), "dtype": "bf16",
        "data": "synthetic: random weights, uniform random token ids",
        "config": {"model": "Qwen3-32B shape", "layers": cfg["num_hidden_layers"], "layers_full": QWEN3_32B["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "intermediate": cfg["intermediate_size"], "global_batch": B, "seq_len": CTX, "page_size": PAGE,
                   "prompt_portion": PORTION, "weight_gb": round(weight_bytes / 1e9, 1)},
        "prefill": {"value": round(CTX / (pf_ms * 1e-3), 1), "tokens": CTX, "portions": CTX // PORTION, "ms": round(pf_ms, 2),
                    "frac": round(pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
        "gpu_launches": launches, "clocks": clocks.summary(c0, c1), "impl": "ours"}))
    return 0


def workload_sweep(args):
    """Qwen3-8B sizes: the decode step at several batch sizes and context lengths (bytes it has to read / time against the
    measured copy bandwidth) and the prefill of one prompt of several lengths, fed in portions of at most 8,192 tokens
    (flops / time against the measured bf16 peak).  One JSON line."""
    import torch

    from mini_sglang_b200 import Engine, EngineArgs
    from mini_sglang_b200.engine.step import StepEntry
    cfg = dict(QWEN3_8B)
    cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    PAGE, W, K = 16, 5, 24
    V = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(0)

    def rand_tokens(n):
        return torch.randint(0, V, (n,), generator=gen).tolist()

    clocks = ClockSampler()
    clocks.start()
    eng = Engine(EngineArgs(model=_write_config(cfg), dummy_load=True, random_seed=0, page_size=PAGE, num_pages=34000,
                            max_num_reqs=66, max_context_len=32768 + 64, max_prefill_tokens=8192, chunk_size=8192,
                            disable_radix_cache=True, schedule_policy="fcfs", log_level="WARNING"))
    runner = eng.runner
    _, weight_bytes, kv_tok = model_sizes(cfg)
    decode, prefill = [], []
    for batch, ctx in ((1, 1024), (1, 4096), (1, 32768), (8, 1024), (8, 4096), (8, 16384), (8, 32768), (64, 1024), (64, 4096), (64, 8192)):
        prompt_len = ctx - (W + K) - 1
        slots = [runner.open() for _ in range(batch)]
        for s in slots:
            toks = rand_tokens(prompt_len)
            for i in range(0, prompt_len, 8192):
                runner.step([StepEntry(s, toks[i:i + 8192], [])])
        feed = [[rand_tokens(1) for _ in slots] for _ in range(W + K)]
        for i in range(W):
            runner.step([StepEntry(s, t, [0]) for s, t in zip(slots, feed[i])])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(W, W + K):
            runner.step([StepEntry(s, t, [0]) for s, t in zip(slots, feed[i])])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / K
        for s in slots:
            runner.close(s)
        need = weight_bytes + batch * (ctx - K // 2) * kv_tok
        decode.append({"batch": batch, "context": ctx, "ms_per_step": round(ms, 3), "tokens_per_s": round(batch / ms * 1e3, 1),
                       "hbm_frac": round(need / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)})
    for n in (512, 2048, 8192, 16384):
        times = []
        for rep in range(4):
            toks = rand_tokens(n)
            s = runner.open()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(0, n, 8192):
                runner.step([StepEntry(s, toks[i:i + 8192], [min(8192, n - i) - 1] if i + 8192 >= n else [])])
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
            runner.close(s)
        ms = sorted(times[1:])[1]
        flops = sum(step_flops(cfg, [min(8192, n - i)], [min(n, i + 8192)], 1 if i + 8192 >= n else 0) for i in range(0, n, 8192))
        prefill.append({"tokens": n, "ms": round(ms, 3), "tokens_per_s": round(n / ms * 1e3, 1),
                        "bf16_frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 3)})
    clocks.stop()
    print(json.dumps({"workload": "sweep", "model": "Qwen3-8B shape", "layers": cfg["num_hidden_layers"], "dtype": "bf16", "page_size": PAGE,
                      "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk["source"]},
                      "decode": decode, "prefill": prefill, "clocks": clocks.summary(), "impl": "ours"}))
    return 0


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
    ap.add_argument("--workload", default="headline", choices=["headline", "qwen3_0.6b_mixed", "qwen3_32b_long", "sweep"],
                    help="headline: the line the contract names; the others: further workloads, one JSON line each")
    ap.add_argument("--skip-sanity", action="store_true", help="no comparison with the plain implementation before timing")
    ap.add_argument("--model", default="8b", choices=["8b", "32b", "0.6b"], help="layer sizes for --only decode / prefill")
    ap.add_argument("--lengths", default=None,
                    help="--only decode: context lengths of the requests instead of --batch x --context: 'lo:hi' spreads --batch "
                         "requests evenly from lo to hi, '30000,1000x15' lists them (x: repeated)")
    ap.add_argument("--kernel-times", action="store_true",
                    help="--only decode: three more steps under the CUDA profiler; the line gets the kernels' mean times")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures the single-GPU engine; --gpus {args.gpus} is not supported (this engine has no multi-GPU path)")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.workload == "qwen3_0.6b_mixed":
        return workload_mixed(args)
    if args.workload == "qwen3_32b_long":
        return workload_long(args)
    if args.workload == "sweep":
        return workload_sweep(args)

    import torch

    from mini_sglang_b200 import Engine, EngineArgs, ops
    from mini_sglang_b200.engine.step import StepEntry

    W, K = max(args.warmup, 3), args.steps
    B, CTX, PAGE, PREFILL = args.batch, args.context, 16, 2048
    SETTLE = 0 if args.only != "all" else 25
    cfg = dict(QWEN3_8B)
    lengths = None
    if args.only != "all":
        cfg = dict({"8b": QWEN3_8B, "32b": QWEN3_32B, "0.6b": QWEN3_0_6B}[args.model])
        if args.lengths:
            lengths = parse_lengths(args.lengths, B)
            B, CTX = len(lengths), max(lengths)
        cfg["max_position_embeddings"] = max(cfg.get("max_position_embeddings", 0), CTX + 64)
    cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    tmp = tempfile.mkdtemp(prefix="msgl_bench_")
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(cfg, f)
    if args.only != "all":
        args.skip_points = True
    max_b = B if args.skip_points else max(B, 64)
    pages = max_b * (CTX // PAGE + 2) + 256
    if lengths:
        pages = sum(n // PAGE + 2 for n in lengths) + 256
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

    layer_params, weight_bytes, kv_bytes_per_token = model_sizes(cfg)
    sanity = None
    if args.only == "all" and not args.skip_sanity:
        sanity = sanity_check(cfg, PAGE)

    clocks = ClockSampler()
    clocks.start()

    def timed_decode(batch, steps, warm, prompt_len=None):
        """Feed given tokens: `batch` requests at context CTX - (warm + steps) .. CTX, or from prompt_len on.  The prompts are
        fed at the power cap and the SM clock needs some 15 decode steps to come back, so SETTLE untimed steps run before the
        `warm` warm-up steps (both are untimed; the timed region is exactly `steps` steps)."""
        warm = warm + SETTLE
        if prompt_len is None:
            prompt_len = CTX - (warm + steps) - 1
        slots = [runner.open() for _ in range(batch)]
        for r, s in enumerate(slots):                             # prompts in portions of 2,048
            n = max(lengths[r] - (warm + steps) - 1, 1) if lengths else prompt_len
            toks = rand_tokens(n)
            for i in range(0, n, 2048):
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
        if args.kernel_times and args.only == "decode":
            kernel_times.update(profile_kernels(lambda: runner.step([StepEntry(s, rand_tokens(1), [0]) for s in slots]), 3,
                                                captures=lambda: len(runner._graphs)))
        for s in slots:
            runner.close(s)
        return ms, launches, (c0, c1)

    kernel_times = {}

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
        line = {"only": "decode", "model": args.model, "layers": L, "batch": B, "context": CTX, "ms_per_step": round(ms_step, 4),
                "launches": launches, "plan": {k: (v if k != "nsplits" else [max(ns) for ns in v]) for k, v in runner.last_plan.items()}}
        if lengths:
            line["lengths"] = args.lengths
        if kernel_times:
            line["kernels"] = kernel_times
        print(json.dumps(line))
        return 0
    value = B / (ms_step * 1e-3)
    step_bytes = weight_bytes + B * (CTX - K // 2) * kv_bytes_per_token
    achieved = step_bytes / (ms_step * 1e-3) / 1e9

    # ---- end to end through the Python entry point: host tokens in, host tokens out
    # Prompts are prefilled in portions, so the requests get their first token a few steps apart; max_new_tokens
    # leaves room for that, so that none of them finishes inside the timed steps.
    # The prompts of all requests are fed at the power cap, and the first decode steps after that run 5-15 % slower until the
    # SM clock has come back (measured: 4.9 ms falling to 4.25 ms over the first 15 steps); the untimed warm-up of this region is
    # therefore SETTLE steps longer.
    W2 = W + SETTLE
    prompt_len = CTX - (W2 + K) - 16
    reqs = [eng.add_request(input_ids=rand_tokens(prompt_len),
                            sampling_params={"temperature": 0.0, "max_new_tokens": W2 + K + 15, "ignore_eos": True})
            for _ in range(B)]
    while any(len(r.output) == 0 for r in reqs):
        eng.step()
    for _ in range(W2 - 1):
        eng.step()
    torch.cuda.synchronize()
    done0 = sum(len(r.output) for r in reqs)
    t0 = time.perf_counter()
    h2d_sum = 0
    for _ in range(K):
        eng.step()
        h2d_sum += runner.last_h2d_bytes
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    done = sum(len(r.output) for r in reqs) - done0
    assert done == B * K, "a request finished inside the timed steps"
    while not eng.scheduler.idle:
        eng.step()
    h2d = h2d_sum // max(K, 1)
    e2e = {"value": round(done / dt, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B, "warmup": W2}

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            ms_b, _, _ = timed_decode(b, max(K, 32), W)
            points[f"decode_b{b}"] = round(b / (ms_b * 1e-3), 1)
        for b in (1, 8, 64):                      # right after 2,048-token prompts
            ms_b, _, _ = timed_decode(b, max(K, 32), W, prompt_len=PREFILL)
            points[f"decode_b{b}_ctx2048"] = round(b / (ms_b * 1e-3), 1)

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
    pf_flops = step_flops(cfg, [PREFILL], [PREFILL], 1)
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
                   "l2": "inputs larger than L2 (15 GB of weights per step), no flush", "peaks": pk["source"],
                   "settle_steps": SETTLE},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks.summary(c0, c1), "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "sanity": sanity, "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
