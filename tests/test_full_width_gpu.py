"""The engine at the full layer sizes of Qwen3-8B (width 4096, 32/8 heads of 128, feed-forward 12288,
vocabulary 151936) with two layers, against the plain implementation: the kernels' real launch shapes
(vector paths, head size 128, the decode attention and weight-streaming GEMM kernels, CUDA graphs), in
float32 and bfloat16, whole / in portions / decoded one by one / mixed."""

import json

import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu

CFG = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 4096, "hidden_act": "silu", "attention_bias": False, "torch_dtype": "bfloat16",
}


@pytest.fixture(scope="module")
def setup():
    from mini_sglang_b200.config import Qwen3Config
    from mini_sglang_b200.config.qwen3 import build_qwen3_spec
    from mini_sglang_b200.parts import expected_tensors
    from mini_sglang_b200.weights import RandomSource
    spec = build_qwen3_spec(Qwen3Config.from_dict(CFG))
    src = RandomSource(expected_tensors(spec), 7, torch.bfloat16, "cuda")
    weights = {n: src.draw(n) for n in expected_tensors(spec) if src.has(n)}          # bfloat16 on the GPU
    g = torch.Generator().manual_seed(3)
    a = torch.randint(0, CFG["vocab_size"], (150,), generator=g).tolist()
    b = torch.randint(0, CFG["vocab_size"], (90,), generator=g).tolist()
    with torch.no_grad():
        torch.backends.cuda.matmul.allow_tf32 = False
        ref = {"a": P.forward_sequence(CFG, weights, a, device="cuda").cpu(),
               "b": P.forward_sequence(CFG, weights, b, device="cuda").cpu()}
    return spec, {"a": a, "b": b}, ref


def check_row(row, want, dtype):
    """float32: element-wise.  bfloat16: every operand is rounded to 8 mantissa bits (unit roundoff 2^-9); a few
    dozen such roundings per token across two layers leave the final hidden state about 1 % off, which shows in
    each of the 151,936 logits as noise of about 1 % of the logits' spread.  So the bound is statistical: the
    error's rms below 1.5 % of the row's rms, and no single logit further off than 7 times that bound (the largest
    of 152k Gaussian draws sits near 4.7 sigma)."""
    if dtype == "float32":
        torch.testing.assert_close(row, want, rtol=2e-4, atol=2e-4)
        return
    err = row - want
    scale = want.pow(2).mean().sqrt().item()
    rms = err.pow(2).mean().sqrt().item()
    assert rms < 0.015 * scale, f"rms error {rms:.4g} vs logits rms {scale:.4g}"
    assert err.abs().max().item() < 7 * 0.015 * scale, f"max error {err.abs().max().item():.4g} vs logits rms {scale:.4g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_width_all_cuts(setup, dtype):
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    spec, seqs, ref = setup
    runner = ModelRunner.from_random(spec, 7, dtype=dtype, page_size=16, num_pages=40, max_reqs=4)
    a, b = seqs["a"], seqs["b"]
    got = {}

    def step(entries):
        out = runner.step([StepEntry(slot, toks, want) for slot, _, _, toks, want in entries]).float().cpu()
        i = 0
        for _, rid, start, toks, want in entries:
            for w in want:
                got[(rid, start + w)] = out[i]
                i += 1

    sa, sb = runner.open(), runner.open()
    step([(sa, "a", 0, a[:70], [0, 69])])                                    # a portion alone
    step([(sa, "a", 70, a[70:118], [47]), (sb, "b", 0, b[:58], [57])])       # portions of two requests
    for i in range(58, 90):                                                  # b one by one, beside a portion of a at first
        ents = [(sb, "b", i, [b[i]], [0])]
        if i == 58:
            ents.append((sa, "a", 118, a[118:120], [0, 1]))
        step(ents)
    for i in range(120, 150):                                                # a one by one (graph replay)
        step([(sa, "a", i, [a[i]], [0])])
    runner.close(sa)
    runner.close(sb)
    assert len(got) == 2 + 1 + 1 + 32 + 2 + 30
    for (rid, pos), row in sorted(got.items()):
        try:
            check_row(row, ref[rid][pos], dtype)
        except AssertionError as e:
            raise AssertionError(f"{dtype}: request {rid} position {pos}: {e}") from None
    # greedy choices agree with the plain implementation's where its margin is clear
    if dtype == "float32":
        for (rid, pos), row in got.items():
            top2 = ref[rid][pos].topk(2).values
            if top2[0] - top2[1] > 1e-2:
                assert int(row.argmax()) == int(ref[rid][pos].argmax())


def test_full_width_short_portions_after_a_long_context():
    """A long context, then portions of 5, 2 and 12 tokens and single tokens: few blocks over many keys, so
    the step function splits the keys of the runs that fit one decode tile, while runs above that go whole to
    the prefill kernel.  bfloat16, against the plain
    implementation."""
    from mini_sglang_b200.config import Qwen3Config
    from mini_sglang_b200.config.qwen3 import build_qwen3_spec
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    from mini_sglang_b200.parts import expected_tensors
    from mini_sglang_b200.weights import RandomSource
    spec = build_qwen3_spec(Qwen3Config.from_dict(CFG))
    src = RandomSource(expected_tensors(spec), 7, torch.bfloat16, "cuda")
    weights = {n: src.draw(n) for n in expected_tensors(spec) if src.has(n)}
    g = torch.Generator().manual_seed(13)
    toks = torch.randint(0, CFG["vocab_size"], (1100,), generator=g).tolist()
    with torch.no_grad():
        ref = P.forward_sequence(CFG, weights, toks, device="cuda").cpu()
    runner = ModelRunner.from_random(spec, 7, dtype="bfloat16", page_size=16, num_pages=80, max_reqs=2)
    s = runner.open()
    got = {}
    cuts = [(0, 1040), (1040, 1045), (1045, 1047), (1047, 1059)] + [(i, i + 1) for i in range(1059, 1100)]
    for lo, hi in cuts:
        want = [0, hi - lo - 1] if hi - lo > 1 else [0]
        out = runner.step([StepEntry(s, toks[lo:hi], want)]).float().cpu()
        for w, row in zip(want, out):
            got[lo + w] = row
    assert runner.use_cuda_graph
    for pos, row in sorted(got.items()):
        try:
            check_row(row, ref[pos], "bfloat16")
        except AssertionError as e:
            raise AssertionError(f"position {pos}: {e}") from None


def test_full_width_one_long_request_among_many_short_ones():
    """64 requests of 18 tokens and one of 1,190 decode together: the blocks of the short ones fill the GPU, so
    nothing would be split for want of blocks, but the long request's keys are many times the mean load of a
    block; the step function cuts them up and replays the graph that has room for the pieces.  bfloat16, the
    long request and two of the short ones against the plain implementation."""
    from mini_sglang_b200.config import Qwen3Config
    from mini_sglang_b200.config.qwen3 import build_qwen3_spec
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    from mini_sglang_b200.parts import expected_tensors
    from mini_sglang_b200.weights import RandomSource
    spec = build_qwen3_spec(Qwen3Config.from_dict(CFG))
    src = RandomSource(expected_tensors(spec), 7, torch.bfloat16, "cuda")
    weights = {n: src.draw(n) for n in expected_tensors(spec) if src.has(n)}
    g = torch.Generator().manual_seed(29)
    n_short, short_len, long_len, n_dec = 64, 18, 1190, 6
    long_toks = torch.randint(0, CFG["vocab_size"], (long_len + n_dec,), generator=g).tolist()
    short_toks = [torch.randint(0, CFG["vocab_size"], (short_len + n_dec,), generator=g).tolist() for _ in range(n_short)]
    with torch.no_grad():
        ref_long = P.forward_sequence(CFG, weights, long_toks, device="cuda").cpu()
        ref_short = {i: P.forward_sequence(CFG, weights, short_toks[i], device="cuda").cpu() for i in (0, n_short - 1)}
    runner = ModelRunner.from_random(spec, 7, dtype="bfloat16", page_size=16, num_pages=2 * n_short + 80, max_reqs=n_short + 2)
    s_long = runner.open()
    runner.step([StepEntry(s_long, long_toks[:long_len], [])])
    shorts = [runner.open() for _ in range(n_short)]
    runner.step([StepEntry(s, t[:short_len], []) for s, t in zip(shorts, short_toks)])
    for i in range(n_dec):
        ents = [StepEntry(s_long, [long_toks[long_len + i]], [0])]
        ents += [StepEntry(s, [t[short_len + i]], [0]) for s, t in zip(shorts, short_toks)]
        out = runner.step(ents).float().cpu()
        for row, want, name in ((out[0], ref_long[long_len + i], "long"), (out[1], ref_short[0][short_len + i], "short 0"),
                                (out[n_short], ref_short[n_short - 1][short_len + i], "last short")):
            try:
                check_row(row, want, "bfloat16")
            except AssertionError as e:
                raise AssertionError(f"decode step {i}, {name} request: {e}") from None
    assert any(wide for _, _, wide in runner._graphs), "the batch should have taken the graph with room for more pieces"


def test_whole_step_decode_kernel_against_plain(monkeypatch):
    """The one-kernel decode step (csrc/decode_step.cu; off by default, forced on here) at Qwen3-8B's widths: 1, 3 and 8
    requests of different lengths decode together, with kv splits, against the plain implementation; and the model must
    really have taken that kernel (one launch per step)."""
    from mini_sglang_b200 import ops
    from mini_sglang_b200.config import Qwen3Config
    from mini_sglang_b200.config.qwen3 import build_qwen3_spec
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    from mini_sglang_b200.parts import expected_tensors
    from mini_sglang_b200.weights import RandomSource
    monkeypatch.setattr(ops, "USE_FUSED_DECODE", True)
    spec = build_qwen3_spec(Qwen3Config.from_dict(CFG))
    src = RandomSource(expected_tensors(spec), 7, torch.bfloat16, "cuda")
    weights = {n: src.draw(n) for n in expected_tensors(spec) if src.has(n)}
    g = torch.Generator().manual_seed(31)
    lens = [1500, 40, 700, 17, 260, 90, 5, 1023]
    n_dec = 5
    seqs = [torch.randint(0, CFG["vocab_size"], (n + n_dec,), generator=g).tolist() for n in lens]
    runner = ModelRunner.from_random(spec, 7, dtype="bfloat16", page_size=16, num_pages=sum(-(-(n + n_dec) // 16) for n in lens) + 8, max_reqs=8)
    assert runner.model.fused_decode is not None
    slots = [runner.open() for _ in lens]
    for s, toks, n in zip(slots, seqs, lens):
        runner.step([StepEntry(s, toks[:n], [])])
    got, fed = {}, [0] * len(lens)
    for live in ([0], [0, 1, 2], list(range(8)), list(range(8)), list(range(8))):
        ents = [StepEntry(slots[i], [seqs[i][lens[i] + fed[i]]], [0]) for i in live]
        out = runner.step(ents).float().cpu()
        assert runner.last_step_used_graph
        for i, row in zip(live, out):
            got[(i, fed[i])] = row
            fed[i] += 1
    assert sorted(k[0] for k in runner._graphs) == [1, 4, 8]
    assert all(gr.n_kernels == 1 for gr in runner._graphs.values()), "the steps did not go through the one-kernel path"
    ops.check_kernel_status()
    assert max(max(ns) for ns in runner.last_plan["nsplits"]) > 1
    for i in range(len(lens)):
        rows = sorted(k for (j, k) in got if j == i)
        with torch.no_grad():
            ref = P.forward_sequence(CFG, weights, seqs[i], device="cuda", rows=[lens[i] + k for k in rows]).cpu()
        for k, want in zip(rows, ref):
            try:
                check_row(got[(i, k)], want, "bfloat16")
            except AssertionError as e:
                raise AssertionError(f"request {i} ({lens[i]} tokens), decoded token {k}: {e}") from None


@pytest.mark.parametrize("shape", [
    ("0.6B", 1024, 16, 8, 3072, True), ("1.7B", 2048, 16, 8, 6144, True), ("4B", 2560, 32, 8, 9728, True),
    ("14B", 5120, 40, 8, 17408, False), ("32B", 5120, 64, 8, 25600, False)], ids=lambda s: s[0])
def test_layer_widths_of_the_other_qwen3_sizes(shape):
    """Two layers at the widths of every other Qwen3 dense size (groups of 2, 4, 5 and 8 query heads per kv head, widths and
    feed-forward widths that are no power of two, tied and untied heads): a 300-token prompt in one step, a 40-token portion,
    two requests decoding through the graph; bfloat16 against the plain implementation."""
    from mini_sglang_b200.config import Qwen3Config
    from mini_sglang_b200.config.qwen3 import build_qwen3_spec
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    from mini_sglang_b200.parts import expected_tensors
    from mini_sglang_b200.weights import RandomSource
    _, H, n_q, n_kv, I, tied = shape
    cfg = dict(CFG, hidden_size=H, num_attention_heads=n_q, num_key_value_heads=n_kv, intermediate_size=I, tie_word_embeddings=tied)
    spec = build_qwen3_spec(Qwen3Config.from_dict(cfg))
    src = RandomSource(expected_tensors(spec), 7, torch.bfloat16, "cuda")
    weights = {n: src.draw(n) for n in expected_tensors(spec) if src.has(n)}
    g = torch.Generator().manual_seed(H + I)
    a = torch.randint(0, cfg["vocab_size"], (346,), generator=g).tolist()
    b = torch.randint(0, cfg["vocab_size"], (25,), generator=g).tolist()
    runner = ModelRunner.from_random(spec, 7, dtype="bfloat16", page_size=16, num_pages=40, max_reqs=2)
    sa, sb = runner.open(), runner.open()
    got = {}
    out = runner.step([StepEntry(sa, a[:300], [0, 299])]).float().cpu()
    got[("a", 0)], got[("a", 299)] = out[0], out[1]
    out = runner.step([StepEntry(sa, a[300:340], [39]), StepEntry(sb, b[:19], [18])]).float().cpu()
    got[("a", 339)], got[("b", 18)] = out[0], out[1]
    for t in range(6):
        out = runner.step([StepEntry(sa, [a[340 + t]], [0]), StepEntry(sb, [b[19 + t]], [0])]).float().cpu()
        assert runner.last_step_used_graph
        got[("a", 340 + t)], got[("b", 19 + t)] = out[0], out[1]
    with torch.no_grad():
        ref = {"a": P.forward_sequence(cfg, weights, a, device="cuda").cpu(), "b": P.forward_sequence(cfg, weights, b, device="cuda").cpu()}
    for (rid, pos), row in sorted(got.items()):
        try:
            check_row(row, ref[rid][pos], "bfloat16")
        except AssertionError as e:
            raise AssertionError(f"{shape[0]}: request {rid} position {pos}: {e}") from None
    runner.close(sa)
    runner.close(sb)
