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
TOL = {"float32": dict(rtol=1e-4, atol=5e-5)}
# bfloat16: every activation between kernels is rounded to 8 mantissa bits (unit roundoff 2^-9), a few dozen
# roundings between the tokens and a logit; they add up to noise of well under one per cent of the logits'
# spread.  The bound is taken against the row's own size, so that it stays able to fail: at these tiny models
# ONE wrong context token among 60 moves the last row by 2.3 % (A) to 5 % (C) of its rms
# (tests/test_plain.py::test_bfloat16_bound_rejects_a_wrong_context_token), and an element-wise bound loose enough
# for the largest logit's rounding would let that pass.
BF16_RMS_FRACTION = 0.015         # rms of the error against the rms of the row
BF16_MAX_FACTOR = 6.0             # no single logit further off than this many times the rms bound
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


def assert_row_close(row: torch.Tensor, want: torch.Tensor, dtype: str) -> None:
    """float32: element-wise.  bfloat16: the error's rms and its largest element, both against the rms of the
    expected row (see BF16_RMS_FRACTION)."""
    if dtype == "float32":
        torch.testing.assert_close(row, want, **TOL["float32"])
        return
    row, want = row.float(), want.float()
    if not torch.isfinite(row).all():
        raise AssertionError("logits are not finite")
    err = row - want
    scale = want.pow(2).mean().sqrt().item()
    rms = err.pow(2).mean().sqrt().item()
    worst = err.abs().max().item()
    if rms > BF16_RMS_FRACTION * scale:
        raise AssertionError(f"rms error {rms:.4g} is {rms / scale:.2%} of the row's rms {scale:.4g} (bound {BF16_RMS_FRACTION:.1%})")
    if worst > BF16_MAX_FACTOR * BF16_RMS_FRACTION * scale:
        raise AssertionError(f"largest error {worst:.4g} is {worst / scale:.2%} of the row's rms {scale:.4g} "
                             f"(bound {BF16_MAX_FACTOR * BF16_RMS_FRACTION:.1%})")


def assert_rows_close(got: torch.Tensor, want: torch.Tensor, dtype: str) -> None:
    """Row by row over the last dimension."""
    assert got.shape == want.shape, f"shape {tuple(got.shape)} against {tuple(want.shape)}"
    g2, w2 = got.reshape(-1, got.shape[-1]), want.reshape(-1, want.shape[-1])
    for i in range(g2.shape[0]):
        try:
            assert_row_close(g2[i], w2[i], dtype)
        except AssertionError as e:
            raise AssertionError(f"row {i}: {e}") from None


def check_against_plain(name: str, dtype: str, got: Dict[tuple, torch.Tensor], seqs: Dict[str, Sequence[int]]):
    ref = {rid: plain_logits(name, toks) for rid, toks in seqs.items()}
    worst = 0.0
    for (rid, pos), row in sorted(got.items()):
        want = ref[rid][pos]
        err = (row - want).abs().max().item()
        worst = max(worst, err)
        try:
            assert_row_close(row, want, dtype)
        except AssertionError as e:
            raise AssertionError(f"request {rid!r} position {pos} ({dtype}, config {name}): {e}") from None
    return worst
