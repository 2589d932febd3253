"""The plain implementation against the reference project's own model code (goldens made by
tests/golden/make_golden.py on the CPU) and against itself in float64."""

import os

import pytest
import torch

import plain_qwen3 as P
from tiny_models import CONFIGS, make_weights

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SEEDS = {"A": 0, "B": 1, "C": 2}


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_plain_matches_reference_goldens(name):
    g = torch.load(os.path.join(GOLD, f"ref_{name}.pt"))
    w = make_weights(CONFIGS[name], SEEDS[name])
    logits = P.forward_sequence(CONFIGS[name], w, g["tokens"])
    torch.testing.assert_close(logits, g["logits"], rtol=1e-5, atol=2e-6)


def test_plain_float64_agrees():
    cfg, w = CONFIGS["B"], make_weights(CONFIGS["B"], 1)
    toks = list(range(3, 40))
    a = P.forward_sequence(cfg, w, toks)
    b = P.forward_sequence(cfg, w, toks, dtype=torch.float64)
    torch.testing.assert_close(a.double(), b, rtol=1e-4, atol=1e-5)


def test_causality_and_prefix_independence():
    cfg, w = CONFIGS["A"], make_weights(CONFIGS["A"], 0)
    toks = [5, 9, 200, 31, 77, 1, 2, 3]
    full = P.forward_sequence(cfg, w, toks)
    part = P.forward_sequence(cfg, w, toks[:5])
    torch.testing.assert_close(full[:5], part, rtol=1e-5, atol=1e-6)


def test_window_attention_plain():
    torch.manual_seed(0)
    q, k, v = torch.randn(9, 4, 8), torch.randn(9, 2, 8), torch.randn(9, 2, 8)
    full = P.causal_gqa_attention(q, k, v, 0.3)
    wide = P.causal_gqa_attention(q, k, v, 0.3, window=100)
    torch.testing.assert_close(full, wide)
    w1 = P.causal_gqa_attention(q, k, v, 0.3, window=1)
    torch.testing.assert_close(w1, v.repeat_interleave(2, dim=1))


def test_philox_known_answer():
    # Random123 known-answer test for Philox4x32-10
    assert P.philox4x32((0, 0, 0, 0), (0, 0)) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert P.philox4x32((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]


def test_sampling_plain():
    logits = torch.tensor([[0.0, 5.0, 1.0], [2.0, 1.0, 0.0]])
    t = torch.tensor([0.0, 1.0])
    noise = torch.tensor([[1.0, 1.0, 1.0], [10.0, 0.01, 10.0]])
    assert P.sample_with_noise(logits, t, noise).tolist() == [1, 1]


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_bfloat16_bound_rejects_a_wrong_context_token(name):
    """The bound that the bfloat16 engine tests use must be able to fail: the logits of the same sequence with ONE
    context token replaced (what reading one wrong, live cache slot looks like), at whichever of 59 places moves
    the last row least, are rejected; so are two neighbouring pages (of two tokens at least) swapped; the right logits with noise of the
    size that bfloat16 rounding leaves are accepted."""
    from helpers import BF16_RMS_FRACTION, PAGE, assert_row_close
    from tiny_models import random_tokens
    cfg, w = CONFIGS[name], make_weights(CONFIGS[name], SEEDS[name])
    toks = random_tokens(60, cfg["vocab_size"], 5)
    with torch.no_grad():
        want = P.forward_sequence(cfg, w, toks)[-1]
        for i in range(59):
            wrong = list(toks)
            wrong[i] = (wrong[i] + 17) % cfg["vocab_size"]
            row = P.forward_sequence(cfg, w, wrong)[-1]
            with pytest.raises(AssertionError):
                assert_row_close(row, want, "bfloat16")
        page = max(PAGE[name], 2)
        for first in range(0, 59 - 2 * page, page):
            wrong = toks[:first] + toks[first + page:first + 2 * page] + toks[first:first + page] + toks[first + 2 * page:]
            if wrong == toks:
                continue
            row = P.forward_sequence(cfg, w, wrong)[-1]
            with pytest.raises(AssertionError):
                assert_row_close(row, want, "bfloat16")
    g = torch.Generator().manual_seed(1)
    noise = torch.randn(want.shape, generator=g) * (0.5 * BF16_RMS_FRACTION * want.pow(2).mean().sqrt())
    assert_row_close(want + noise, want, "bfloat16")
    assert_row_close(want, want, "float32")
    with pytest.raises(AssertionError):
        assert_row_close(want + 1e-3, want, "float32")
