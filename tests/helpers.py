"""Shared helpers of the GPU tests: model folders in temporary directories, plain-implementation
logits, and a driver that feeds a trace (list of steps) to a ModelRunner."""

from __future__ import annotations

import functools
import os
import tempfile
from typing import Dict, List, Sequence

import torch

import plain_qwen3
from tiny_models import CONFIGS, make_weights, write_model_dir

SEEDS = {"A": 0, "B": 1, "C": 2}
PAGE = {"A": 1, "B": 4, "C": 16}
TOL = {"float32": dict(rtol=1e-4, atol=5e-5), "bfloat16": dict(rtol=3e-2, atol=3e-2)}
_tmp = tempfile.TemporaryDirectory(prefix="msgl_models_")


@functools.lru_cache(None)
def model_dir(name: str) -> str:
    d = os.path.join(_tmp.name, name)
    write_model_dir(d, CONFIGS[name], make_weights(CONFIGS[name], SEEDS[name]))
    return d


@functools.lru_cache(None)
def weights(name: str):
    return make_weights(CONFIGS[name], SEEDS[name])


def plain_logits(name: str, tokens: Sequence[int]) -> torch.Tensor:
    with torch.no_grad():                      # on the CPU: IEEE float32, no device-specific roundings
        return plain_qwen3.forward_sequence(CONFIGS[name], weights(name), list(tokens), device="cpu")


def make_runner(name: str, dtype: str, num_pages: int, max_reqs: int = 4, page_size: int = None, graphs: bool = True):
    from mini_sglang_b200.engine.step import ModelRunner
    return ModelRunner.from_model_dir(model_dir(name), dtype=dtype, page_size=page_size or PAGE[name],
                                      num_pages=num_pages, max_reqs=max_reqs, use_cuda_graph=graphs)


def play(runner, steps: List[dict]) -> Dict[tuple, torch.Tensor]:
    """steps: [{"entries": [(rid, tokens, want)], "end": [rid]}] -> {(rid, position): logits row}."""
    from mini_sglang_b200.engine.step import StepEntry
    slots, fed, got = {}, {}, {}
    for st in steps:
        entries, keys = [], []
        for rid, toks, want in st["entries"]:
            if rid not in slots:
                slots[rid] = runner.open()
                fed[rid] = 0
            entries.append(StepEntry(slots[rid], toks, want))
            keys.extend((rid, fed[rid] + w) for w in want)
            fed[rid] += len(toks)
        logits = runner.step(entries).float().cpu()
        assert logits.shape[0] == len(keys)
        for k, row in zip(keys, logits):
            got[k] = row
        for rid in st.get("end", []):
            runner.close(slots.pop(rid))
    for rid in list(slots):
        runner.close(slots.pop(rid))
    return got


def check_against_plain(name: str, dtype: str, got: Dict[tuple, torch.Tensor], seqs: Dict[str, Sequence[int]]):
    ref = {rid: plain_logits(name, toks) for rid, toks in seqs.items()}
    worst = 0.0
    for (rid, pos), row in sorted(got.items()):
        want = ref[rid][pos]
        err = (row - want).abs().max().item()
        worst = max(worst, err)
        try:
            torch.testing.assert_close(row, want, **TOL[dtype])
        except AssertionError as e:
            raise AssertionError(f"request {rid!r} position {pos} ({dtype}, config {name}): {e}") from None
    return worst
