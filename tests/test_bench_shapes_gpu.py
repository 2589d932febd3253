"""The shapes that bench.py times, against the plain implementation: Qwen3-8B's layer widths (two layers), a
2,048-token prompt in one step and a second 2,048-token portion behind it, 8 and 64 requests decoding at about
4,090 keys through the CUDA graphs with the kv splits that the planner chooses by itself, 64 requests beyond
6,144 keys, where the planner halves every request, and one request of 32,000 tokens (portions of 8,192, 32 kv splits).  Each test also asserts which graph and which splits were
taken, so that a change of the planner cannot quietly move the benchmark onto a path that is compared nowhere."""

import pytest
import torch

import plain_qwen3 as P
from helpers import assert_row_close

pytestmark = pytest.mark.gpu

CFG = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 8192, "hidden_act": "silu", "attention_bias": False, "torch_dtype": "bfloat16",
}
PAGE = 16


@pytest.fixture(scope="module")
def model():
    from mini_sglang_b200.config import Qwen3Config
    from mini_sglang_b200.config.qwen3 import build_qwen3_spec
    from mini_sglang_b200.parts import expected_tensors
    from mini_sglang_b200.weights import RandomSource
    spec = build_qwen3_spec(Qwen3Config.from_dict(CFG))
    src = RandomSource(expected_tensors(spec), 11, torch.bfloat16, "cuda")
    weights = {n: src.draw(n) for n in expected_tensors(spec) if src.has(n)}          # bfloat16 on the GPU
    torch.backends.cuda.matmul.allow_tf32 = False
    return spec, weights


def tokens(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, CFG["vocab_size"], (n,), generator=g).tolist()


def plain_rows(weights, toks, rows):
    with torch.no_grad():
        out = P.forward_sequence(CFG, weights, toks, device="cuda", rows=list(rows)).cpu()
    return dict(zip(rows, out))


def close(row, want, dtype, what):
    try:
        if dtype == "float32":
            torch.testing.assert_close(row, want, rtol=2e-4, atol=2e-4)
        else:
            assert_row_close(row, want, dtype)
    except AssertionError as e:
        raise AssertionError(f"{dtype}, {what}: {e}") from None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_of_2048_tokens_in_one_step_and_a_second_portion_behind_it(model, dtype):
    from mini_sglang_b200 import ops
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    spec, weights = model
    toks = tokens(4096, 41)
    runner = ModelRunner.from_random(spec, 11, dtype=dtype, page_size=PAGE, num_pages=4096 // PAGE + 4, max_reqs=2)
    s = runner.open()
    before = ops.LAUNCHES
    want1, want2 = [0, 1, 1023, 2046, 2047], [0, 1, 1000, 2047]
    out1 = runner.step([StepEntry(s, toks[:2048], want1)]).float().cpu()
    out2 = runner.step([StepEntry(s, toks[2048:], want2)]).float().cpu()
    ops.check_kernel_status()
    assert ops.LAUNCHES > before and not runner.last_step_used_graph
    if dtype == "bfloat16":       # the tcgen05 kernels took these steps (a refusal would have switched them off for good)
        assert ops.USE_TC_ATTENTION and ops.TC_VERSION == 2 and ops._tc2_usable
        assert ops.TC_GEMM in ("swiglu", "all") and ops.TC_GEMM_CTAS == 2 and ops._tc_gemm_usable
    ref = plain_rows(weights, toks, want1 + [2048 + w for w in want2])
    for w, row in zip(want1, out1):
        close(row, ref[w], dtype, f"first portion, place {w}")
    for w, row in zip(want2, out2):
        close(row, ref[2048 + w], dtype, f"second portion, place {w} (position {2048 + w})")
    runner.close(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_eight_requests_decode_at_4090_keys_with_the_planners_splits(model, dtype):
    from mini_sglang_b200 import ops
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    spec, weights = model
    n_req, n_ctx, n_dec = 8, 4088, 8
    seqs = [tokens(n_ctx + n_dec, 50 + i) for i in range(n_req)]
    runner = ModelRunner.from_random(spec, 11, dtype=dtype, page_size=PAGE, num_pages=n_req * (4096 // PAGE) + 4, max_reqs=n_req)
    slots = [runner.open() for _ in range(n_req)]
    got = {}
    for i in range(0, n_req, 2):                           # two prompts a step: 8,176 tokens
        out = runner.step([StepEntry(slots[j], seqs[j][:n_ctx], [n_ctx - 1]) for j in (i, i + 1)]).float().cpu()
        got[(i, n_ctx - 1)], got[(i + 1, n_ctx - 1)] = out[0], out[1]
    for t in range(n_dec):
        out = runner.step([StepEntry(slots[j], [seqs[j][n_ctx + t]], [0]) for j in range(n_req)]).float().cpu()
        assert runner.last_step_used_graph
        for j in range(n_req):
            got[(j, n_ctx + t)] = out[j]
        if dtype == "bfloat16":
            # 4 blocks an SM x 148 SMs over 8 requests x 8 kv heads leave room for 9 pieces a request; 4,096 keys are
            # 256 units of 16 for 4 warps, which 8 blocks share as evenly as 9
            assert runner.last_plan["graph_key"] == (8, (256,), False), runner.last_plan
            assert runner.last_plan["nsplits"] == [[8] * n_req], runner.last_plan
        else:
            assert runner.last_plan["graph_key"][0] == 8 and min(runner.last_plan["nsplits"][0]) > 1, runner.last_plan
    ops.check_kernel_status()
    for j in range(n_req):
        rows = list(range(n_ctx - 1, n_ctx + n_dec))
        ref = plain_rows(weights, seqs[j], rows)
        for r in rows:
            close(got[(j, r)], ref[r], dtype, f"request {j}, position {r}")
    for s in slots:
        runner.close(s)


def test_sixtyfour_requests_decode_at_4090_keys_and_beyond_6144(model):
    """bfloat16.  64 requests x 8 kv heads are 512 blocks, 3.5 an SM: at 4,090 keys nothing is cut (the narrow graph),
    beyond 6,144 keys every request is halved (the graph with room for more pieces).  Between the two, every request is
    fed a 2,100-token portion behind its 4,092 cached tokens (the tcgen05 prefill kernel over a long prefix)."""
    from mini_sglang_b200 import ops
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    spec, weights = model
    dtype = "bfloat16"
    n_req, n_ctx, n_dec, n_more, n_dec2 = 64, 4088, 4, 2100, 3
    total = n_ctx + n_dec + n_more + n_dec2
    seqs = [tokens(total, 100 + i) for i in range(n_req)]
    checked = [0, 1, 31, 62, 63]
    runner = ModelRunner.from_random(spec, 11, dtype=dtype, page_size=PAGE, num_pages=n_req * (-(-total // PAGE)) + 4, max_reqs=n_req)
    slots = [runner.open() for _ in range(n_req)]
    got = {}
    for i in range(0, n_req, 2):
        runner.step([StepEntry(slots[j], seqs[j][:n_ctx], []) for j in (i, i + 1)])
    pos = n_ctx
    for t in range(n_dec):
        out = runner.step([StepEntry(slots[j], [seqs[j][pos]], [0]) for j in range(n_req)]).float().cpu()
        assert runner.last_step_used_graph
        assert runner.last_plan["graph_key"] == (64, (256,), False) and runner.last_plan["nsplits"] == [[1] * n_req], runner.last_plan
        for j in checked:
            got[(j, pos)] = out[j]
        pos += 1
    for i in range(0, n_req, 3):                           # three portions a step: 6,300 tokens
        js = [j for j in (i, i + 1, i + 2) if j < n_req]
        out = runner.step([StepEntry(slots[j], seqs[j][pos:pos + n_more], [0, n_more - 1]) for j in js]).float().cpu()
        for k, j in enumerate(js):
            if j in checked:
                got[(j, pos)], got[(j, pos + n_more - 1)] = out[2 * k], out[2 * k + 1]
    pos += n_more
    assert pos >= 6144 + 48
    for t in range(n_dec2):
        out = runner.step([StepEntry(slots[j], [seqs[j][pos]], [0]) for j in range(n_req)]).float().cpu()
        assert runner.last_step_used_graph
        assert runner.last_plan["graph_key"] == (64, (512,), True) and runner.last_plan["nsplits"] == [[2] * n_req], runner.last_plan
        for j in checked:
            got[(j, pos)] = out[j]
        pos += 1
    ops.check_kernel_status()
    for j in checked:
        rows = sorted(r for (jj, r) in got if jj == j)
        assert len(rows) == n_dec + 2 + n_dec2
        ref = plain_rows(weights, seqs[j], rows)
        for r in rows:
            close(got[(j, r)], ref[r], dtype, f"request {j}, position {r}")
    for s in slots:
        runner.close(s)


def test_one_request_of_32000_tokens(model):
    """A long context: 32,000 tokens fed in portions of 8,192 (the tcgen05 prefill kernel over prefixes of up to 24,576 keys),
    then decoded token by token with the keys cut into 32 pieces (the decode graph with the wide split dimension).  bfloat16,
    the last row of every portion and every decoded row against the plain implementation."""
    from mini_sglang_b200 import ops
    from mini_sglang_b200.config import Qwen3Config
    from mini_sglang_b200.config.qwen3 import build_qwen3_spec
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    _, weights = model
    cfg = dict(CFG, max_position_embeddings=32768)
    spec = build_qwen3_spec(Qwen3Config.from_dict(cfg))
    n_ctx, n_dec = 32000, 3
    toks = tokens(n_ctx + n_dec, 77)
    runner = ModelRunner.from_random(spec, 11, dtype="bfloat16", page_size=PAGE, num_pages=(n_ctx + n_dec) // PAGE + 8, max_reqs=2)
    s = runner.open()
    got = {}
    for lo in range(0, n_ctx, 8192):
        hi = min(lo + 8192, n_ctx)
        got[hi - 1] = runner.step([StepEntry(s, toks[lo:hi], [hi - lo - 1])]).float().cpu()[0]
    for t in range(n_dec):
        got[n_ctx + t] = runner.step([StepEntry(s, [toks[n_ctx + t]], [0])]).float().cpu()[0]
        assert runner.last_step_used_graph
        assert runner.last_plan["graph_key"] == (1, (2048,), True) and runner.last_plan["nsplits"] == [[32]], runner.last_plan
    ops.check_kernel_status()
    rows = sorted(got)
    with torch.no_grad():
        ref = P.forward_sequence(cfg, weights, toks, device="cuda", rows=rows).cpu()
    for r, want in zip(rows, ref):
        close(got[r], want, "bfloat16", f"position {r}")
    runner.close(s)
