"""The Python entry point, in the manner of the reference's Engine
(mini_sglang/entrypoints/engine.py:19-99, usage in its example.py): construct from the
arguments, then `generate(prompt | input_ids, sampling_params, stream)`.

This engine is one process: model, cache, scheduler and sampling live in the caller's process
(the reference spawns a scheduler and a detokenizer process and talks to them over ZMQ; that is
server plumbing and out of scope here).  Text prompts need a tokenizer in the model folder;
token ids always work.
"""

from __future__ import annotations

import asyncio
import atexit
import json
import logging
import os
import time
import uuid
from typing import AsyncIterator, Dict, Iterator, List, Optional, Sequence, Union

import torch

from ..config import load_config
from ..sampling import Sampler, SamplingParams
from ..weights import CheckpointSource, RandomSource
from .args import EngineArgs
from .scheduler import Req, Scheduler, StepOutput
from .step import ModelRunner

logger = logging.getLogger("mini_sglang_b200")


def _load_tokenizer(model_dir: str):
    if not any(os.path.isfile(os.path.join(model_dir, f)) for f in ("tokenizer.json", "tokenizer.model", "vocab.json")):
        return None
    try:
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(model_dir, local_files_only=True)
    except Exception as e:          # a broken tokenizer folder must not stop token-id use
        logger.warning("tokenizer in %s could not be loaded (%s); only input_ids are accepted", model_dir, e)
        return None


class Engine:
    def __init__(self, args: EngineArgs):
        self.args = args
        logging.basicConfig(level=getattr(logging, args.log_level, logging.INFO))
        cfg, spec = load_config(args.model)
        self.config, self.spec = cfg, spec
        max_ctx = min(args.max_context_len or spec.max_context_len, spec.max_context_len)
        if args.dummy_load:
            factory = lambda exp, dt, dev: RandomSource(exp, args.random_seed, dt, dev)     # noqa: E731
        else:
            factory = lambda exp, dt, dev: CheckpointSource(args.model, exp, dt, dev)       # noqa: E731
        t0 = time.time()
        self.runner = ModelRunner(spec, factory, dtype=args.dtype, page_size=args.page_size, num_pages=args.num_pages,
                                  max_reqs=args.max_num_reqs, max_context_len=max_ctx,
                                  max_step_tokens=args.max_prefill_tokens,
                                  gpu_memory_utilization=args.gpu_memory_utilization,
                                  use_cuda_graph=not args.disable_cuda_graph, max_capture_bs=args.max_capture_bs)
        self.sampler = Sampler(args.random_seed, self.runner.device)
        self.scheduler = Scheduler(
            self.runner, self.sampler, max_num_reqs=args.max_num_reqs, max_step_tokens=args.max_prefill_tokens,
            chunk_size=args.chunk_size, policy=args.schedule_policy, conservativeness=args.schedule_conservativeness,
            retract_decode_steps=args.retract_decode_steps, enable_prefix_cache=not args.disable_radix_cache,
            eos_ids=spec.eos_token_ids, init_new_token_ratio=args.init_new_token_ratio,
            min_new_token_ratio_factor=args.min_new_token_ratio_factor,
            new_token_ratio_decay_steps=args.new_token_ratio_decay_steps, seed=args.random_seed,
            lookahead=not args.disable_overlap)
        self.tokenizer = _load_tokenizer(args.model)
        self.step_times: List[float] = []
        self.step_records: List[Dict] = []          # --profile: one record per step
        self._profile_written = 0                   # records already saved
        if args.profile:
            from ..parts import model as _model
            _model.NVTX_RANGES = True
            atexit.register(self.write_profile)
        self._load_seconds = time.time() - t0
        logger.info("engine ready in %.1f s: %d cache pages of %d tokens", self._load_seconds,
                    self.runner.mgr.groups[0].pool.num_pages if self.runner.mgr.groups else 0, args.page_size)

    # -- requests --------------------------------------------------------------------------
    def _make_req(self, prompt: Optional[str], input_ids: Optional[Sequence[int]], sampling_params) -> Req:
        if input_ids is None:
            if prompt is None:
                raise ValueError("give either prompt or input_ids")
            if self.tokenizer is None:
                raise ValueError("the model folder has no tokenizer; pass input_ids")
            input_ids = self.tokenizer.encode(prompt)
        input_ids = [int(t) for t in input_ids]
        vocab = self.spec.vocab_size
        bad = [t for t in input_ids if not 0 <= t < vocab]
        if bad:       # refused here: inside a step it would stop every other request of the batch as well
            raise ValueError(f"token id {bad[0]} is outside the model's vocabulary [0, {vocab})")
        import dataclasses as _dc
        params = (_dc.replace(sampling_params) if isinstance(sampling_params, SamplingParams)
                  else SamplingParams.init_from_dict(sampling_params))
        return Req(uuid.uuid4().hex, input_ids, params, self.spec.eos_token_ids)

    def add_request(self, prompt=None, sampling_params=None, input_ids=None) -> Req:
        req = self._make_req(prompt, input_ids, sampling_params)
        self.scheduler.add_request(req)
        return req

    def step(self) -> List[StepOutput]:
        """One scheduler step: the public unit of work (a batch through the model, sampling,
        bookkeeping).  Returns what each sampled request got; unless args.disable_overlap, these are the
        tokens of the step that the call before launched (they travel to the host while the next step runs).

        With args.profile every step is bracketed by an NVTX range and two CUDA events, waited for, and
        recorded: what the step held (batch, tokens, prompt tokens, CUDA graph or not), its time on the host
        and on the device, and the number of this engine's kernels it launched; `write_profile` saves the list."""
        if not self.args.profile:
            return self.scheduler.step()
        from .. import ops
        steps_before, launches_before = self.scheduler.stats["steps"], ops.LAUNCHES
        torch.cuda.nvtx.range_push(f"step {steps_before}")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        out = self.scheduler.step()
        e1.record()
        host_ms = (time.perf_counter() - t0) * 1e3
        torch.cuda.synchronize()
        torch.cuda.nvtx.range_pop()
        self.step_times.append(time.perf_counter() - t0)
        if self.scheduler.stats["steps"] > steps_before:          # a batch was launched
            self.step_records.append({**self.scheduler.last_step, "host_ms": round(host_ms, 4),
                                      "device_ms": round(e0.elapsed_time(e1), 4),
                                      "wall_ms": round(self.step_times[-1] * 1e3, 4),
                                      "kernels": ops.LAUNCHES - launches_before, "sampled": len(out)})
        return out

    def write_profile(self, path: Optional[str] = None) -> Optional[str]:
        """Save the per-step records of --profile as JSON (default: traces/steps_<time>_<pid>.json under
        args.profile_dir, as the reference keeps its traces under traces/, mini_sglang/utils/profiler.py:16-58).
        Called at shutdown() and at interpreter exit; a second call without new steps writes nothing."""
        if not self.args.profile or not self.step_records or (path is None and self._profile_written == len(self.step_records)):
            return None
        if path is None:
            os.makedirs(self.args.profile_dir, exist_ok=True)
            path = os.path.join(self.args.profile_dir, f"steps_{time.strftime('%Y%m%d-%H%M%S')}_{os.getpid()}.json")
        kinds = {}
        for r in self.step_records:
            k = kinds.setdefault(r["kind"], {"steps": 0, "tokens": 0, "device_ms": 0.0, "host_ms": 0.0})
            k["steps"] += 1
            k["tokens"] += r["tokens"]
            k["device_ms"] += r["device_ms"]
            k["host_ms"] += r["host_ms"]
        with open(path, "w") as f:
            json.dump({"model": self.args.model, "dtype": self.args.dtype, "page_size": self.args.page_size,
                       "summary": kinds, "scheduler": dict(self.scheduler.stats), "steps": self.step_records}, f)
        self._profile_written = len(self.step_records)
        logger.info("[profile] %d steps written to %s", len(self.step_records), path)
        return path

    def _result(self, req: Req, t_start: float) -> Dict:
        out = req.output
        text = self.tokenizer.decode(out) if self.tokenizer is not None else None
        return {"text": text, "token_ids": list(out),
                "meta_info": {"id": req.rid, "finish_reason": req.finish_reason.to_json() if req.finish_reason else None,
                              "prompt_tokens": req.n_prompt, "completion_tokens": len(out),
                              "cached_tokens": req.cached_tokens, "e2e_latency": time.time() - t_start}}

    def generate(self, prompt: Union[None, str, List[str]] = None, sampling_params: Union[None, Dict, List[Dict]] = None,
                 input_ids: Union[None, List[int], List[List[int]]] = None, stream: bool = False):
        """One request -> dict (or, with stream=True, an iterator of dicts, one per new token);
        a list of prompts or of token-id lists -> a list of dicts, run together as a batch."""
        batch = (isinstance(prompt, (list, tuple))) or (input_ids is not None and len(input_ids) > 0 and isinstance(input_ids[0], (list, tuple)))
        t0 = time.time()
        if not batch:
            req = self.add_request(prompt, sampling_params, input_ids)
            if stream:
                return self._stream(req, t0)
            self._run_until([req])
            return self._result(req, t0)
        if stream:
            raise ValueError("stream=True takes a single request")
        n = len(prompt) if prompt is not None else len(input_ids)
        sp = sampling_params if isinstance(sampling_params, (list, tuple)) else [sampling_params] * n
        reqs = [self.add_request(prompt[i] if prompt is not None else None, sp[i],
                                 input_ids[i] if input_ids is not None else None) for i in range(n)]
        self._run_until(reqs)
        return [self._result(r, t0) for r in reqs]

    def _run_until(self, reqs: Sequence[Req]) -> None:
        while not all(r.finished for r in reqs):
            if self.scheduler.idle:
                raise RuntimeError("scheduler went idle with unfinished requests")
            self.step()

    def _stream(self, req: Req, t0: float) -> Iterator[Dict]:
        sent = 0
        while True:
            if not req.finished:
                self.step()
            if len(req.output) > sent or req.finished:
                sent = len(req.output)
                yield self._result(req, t0)
            if req.finished:
                return

    # -- maintenance -----------------------------------------------------------------------
    def flush_cache(self) -> bool:
        return self.scheduler.flush_cache()

    def get_server_info(self) -> Dict:
        import dataclasses as _dc
        mgr = self.runner.mgr
        return {**_dc.asdict(self.args),
                "internal_states": [{"cache_pages": [g.pool.num_pages for g in mgr.groups],
                                     "free_pages": [g.pool.available for g in mgr.groups],
                                     "cache_bytes": self.runner.storage.bytes(),
                                     "new_token_ratio": self.scheduler.new_token_ratio,
                                     "waiting": len(self.scheduler.waiting), "running": len(self.scheduler.running),
                                     **self.scheduler.stats}]}

    def shutdown(self) -> None:
        """One process: nothing to stop.  Saves the step records of --profile."""
        self.write_profile()

    # -- asyncio face (the reference's Engine.async_generate, mini_sglang/entrypoints/engine.py:63-85) -----
    async def async_generate(self, prompt: Optional[str] = None, sampling_params: Optional[Dict] = None,
                             input_ids: Optional[List[int]] = None, stream: bool = False):
        """`await engine.async_generate(...)` -> dict, or with stream=True an async iterator of dicts, one per
        new token.  Several coroutines may generate at once: their requests run as one batch, whichever coroutine
        happens to hold the engine makes the next step, and every step is followed by a yield to the event loop."""
        req = self.add_request(prompt, sampling_params, input_ids)
        t0 = time.time()
        if stream:
            return self._astream(req, t0)
        while not req.finished:
            self.step()
            await asyncio.sleep(0)
        return self._result(req, t0)

    async def _astream(self, req: Req, t0: float) -> AsyncIterator[Dict]:
        sent = 0
        while True:
            if not req.finished:
                self.step()
                await asyncio.sleep(0)
            if len(req.output) > sent or req.finished:
                sent = len(req.output)
                yield self._result(req, t0)
            if req.finished:
                return
