"""Random small Qwen3 configurations (seeded): head sizes from 16 to 256 in steps of 16, odd head counts and
groups, widths, feed-forward sizes and vocabularies that are no power of two (and not even multiples of 8),
biases, tied heads, page sizes 1..32.  Each is replayed whole, in portions, token by token and mixed with a
second request, in float32 and bfloat16, against the plain implementation."""

import os
import random
import tempfile

import pytest
import torch

import plain_qwen3
from helpers import assert_row_close, play
from tiny_models import make_weights, random_tokens, write_model_dir

pytestmark = pytest.mark.gpu


def random_config(seed: int) -> dict:
    r = random.Random(seed)
    d = 16 * r.randrange(1, 17) if seed % 3 else r.choice([16, 48, 80, 112, 128, 144, 256])
    n_kv = r.choice([1, 2, 3, 5])
    group = r.choice([1, 2, 3, 4, 7]) if d <= 128 else r.choice([1, 2])
    hidden = r.choice([40, 72, 100, 136, 168, 36, 250])
    return {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
        "num_hidden_layers": r.randrange(1, 4), "hidden_size": hidden,
        "num_attention_heads": n_kv * group, "num_key_value_heads": n_kv, "head_dim": d,
        "intermediate_size": r.choice([56, 100, 144, 90, 256]), "vocab_size": r.choice([97, 333, 1003, 256, 515]),
        "rope_theta": r.choice([1e4, 5e4, 1e6]), "rms_norm_eps": r.choice([1e-6, 1e-5, 3e-6]),
        "tie_word_embeddings": r.random() < 0.5, "max_position_embeddings": 1024, "hidden_act": "silu",
        "attention_bias": r.random() < 0.3, "torch_dtype": "bfloat16", "eos_token_id": 1,
    }


@pytest.mark.parametrize("seed", range(10))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configuration(seed, dtype):
    from mini_sglang_b200.engine.step import ModelRunner
    cfg = random_config(seed)
    w = make_weights(cfg, 40 + seed, std=0.05)
    r = random.Random(1000 + seed)
    a = random_tokens(r.randrange(40, 150), cfg["vocab_size"], 1 + seed)
    b = random_tokens(r.randrange(20, 70), cfg["vocab_size"], 2 + seed)
    with torch.no_grad():
        ref = {"a": plain_qwen3.forward_sequence(cfg, w, a, device="cpu"), "b": plain_qwen3.forward_sequence(cfg, w, b, device="cpu")}
    with tempfile.TemporaryDirectory(prefix="msgl_rand_") as tmp:
        write_model_dir(os.path.join(tmp, "m"), cfg, w)
        page = r.choice([1, 4, 8, 16, 32])
        runner = ModelRunner.from_model_dir(os.path.join(tmp, "m"), dtype=dtype, page_size=page,
                                            num_pages=(len(a) + len(b)) // page + 12, max_reqs=3)
        cut = r.randrange(5, len(a) - 20)
        steps = [{"entries": [("a", a[:cut], [0, cut - 1])]}]                                   # a portion
        steps.append({"entries": [("a", a[cut:cut + 2], [1]), ("b", b[:len(b) - 8], [len(b) - 9])]})   # two tokens beside a portion
        pos = cut + 2
        for i in range(len(b) - 8, len(b)):                                                  # b token by token, a in small portions
            ents = [("b", [b[i]], [0])]
            if pos < len(a):
                n = min(r.randrange(1, 7), len(a) - pos)
                ents.append(("a", a[pos:pos + n], [n - 1]))
                pos += n
            steps.append({"entries": ents})
        steps[-1]["end"] = ["b"]
        while pos < len(a):                                                                  # the rest of a one by one (graph replay)
            steps.append({"entries": [("a", [a[pos]], [0])]})
            pos += 1
        got = play(runner, steps)
    assert got
    for (rid, p), row in sorted(got.items()):
        try:
            assert_row_close(row, ref[rid][p], dtype)
        except AssertionError as e:
            raise AssertionError(f"seed {seed} {dtype} config {cfg}: request {rid} position {p}: {e}") from None
