"""Generation through the Python entry point and the command line."""

import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as P
from helpers import PAGE, model_dir, plain_logits, weights
from tiny_models import CONFIGS, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def make_engine(name, dtype, **kw):
    from mini_sglang_b200 import Engine, EngineArgs
    args = dict(model=model_dir(name), dtype=dtype, page_size=PAGE[name], num_pages=256, max_num_reqs=8, random_seed=0,
                log_level="WARNING")
    args.update(kw)
    return Engine(EngineArgs(**args))


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_float32_equals_plain(name):
    cfg = CONFIGS[name]
    eng = make_engine(name, "float32")
    prompts = [random_tokens(n, cfg["vocab_size"], 900 + n) for n in (5, 9, 13)]
    outs = eng.generate(input_ids=prompts, sampling_params={"temperature": 0.0, "max_new_tokens": 8, "ignore_eos": True})
    for p, o in zip(prompts, outs):
        want = P.greedy_generate(cfg, weights(name), p, 8, device="cpu")
        assert o["token_ids"] == want
        assert o["meta_info"]["finish_reason"] == {"type": "length", "length": 8}
        assert o["meta_info"]["prompt_tokens"] == len(p) and o["meta_info"]["completion_tokens"] == 8
    eng.scheduler.check_idle_invariants()


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_bfloat16_follows_plain_logits(name):
    """bfloat16 may break a near-tie differently; every chosen token must be (near-)best under the
    plain implementation given the same history."""
    cfg = CONFIGS[name]
    eng = make_engine(name, "bfloat16")
    p = random_tokens(11, cfg["vocab_size"], 950)
    out = eng.generate(input_ids=p, sampling_params={"max_new_tokens": 12, "ignore_eos": True})
    toks = out["token_ids"]
    ref = plain_logits(name, p + toks)
    for i, t in enumerate(toks):
        row = ref[len(p) - 1 + i]
        assert row[t] >= row.max() - 0.05, (i, t, row[t].item(), row.max().item())


def test_chunked_prefill_budget_and_small_pool_same_tokens():
    name, cfg = "B", CONFIGS["B"]
    prompts = [random_tokens(n, cfg["vocab_size"], 1000 + n) for n in (7, 16, 23, 31, 40, 12)]
    sp = {"temperature": 0.0, "max_new_tokens": 10, "ignore_eos": True}
    base = make_engine(name, "float32", disable_radix_cache=True, schedule_policy="fcfs").generate(input_ids=prompts, sampling_params=sp)
    tight = make_engine(name, "float32", num_pages=24, chunk_size=8, max_prefill_tokens=20, schedule_conservativeness=0.3)
    outs = tight.generate(input_ids=prompts, sampling_params=sp)
    assert [o["token_ids"] for o in outs] == [o["token_ids"] for o in base]
    tight.scheduler.check_idle_invariants()
    assert tight.scheduler.stats["retractions"] > 0 or tight.scheduler.stats["evicted_pages"] > 0


def test_prefix_reuse_gives_same_tokens_and_counts_cached():
    name, cfg = "B", CONFIGS["B"]
    shared = random_tokens(40, cfg["vocab_size"], 1100)        # longer than the 32 tokens that make a request wait
    prompts = [shared + random_tokens(5, cfg["vocab_size"], 1101 + i) for i in range(4)]
    sp = {"max_new_tokens": 6, "ignore_eos": True}
    eng = make_engine(name, "float32")
    outs = eng.generate(input_ids=prompts, sampling_params=sp)
    assert [o["meta_info"]["cached_tokens"] for o in outs] == [0, 40, 40, 40]
    for p, o in zip(prompts, outs):
        assert o["token_ids"] == P.greedy_generate(cfg, weights(name), p, 6, device="cpu")
    # and again, now everything but the last page comes from the cache
    again = eng.generate(input_ids=prompts[0], sampling_params=sp)
    assert again["token_ids"] == outs[0]["token_ids"] and again["meta_info"]["cached_tokens"] == 44
    assert eng.flush_cache()
    eng.scheduler.check_idle_invariants()


def test_temperature_sampling_is_seeded_and_batch_independent():
    name, cfg = "B", CONFIGS["B"]
    prompts = [random_tokens(n, cfg["vocab_size"], 1200 + n) for n in (7, 16, 23, 31)]
    sps = [{"temperature": 0.7, "max_new_tokens": 6, "ignore_eos": True, "seed": 1 + i} for i in range(4)]
    a = make_engine(name, "float32", random_seed=1).generate(input_ids=prompts, sampling_params=sps)
    b = make_engine(name, "float32", random_seed=1, chunk_size=8, max_prefill_tokens=16).generate(input_ids=prompts, sampling_params=sps)
    assert [o["token_ids"] for o in a] == [o["token_ids"] for o in b]
    alone = make_engine(name, "float32", random_seed=1).generate(input_ids=prompts[2], sampling_params=sps[2])
    assert alone["token_ids"] == a[2]["token_ids"]
    other = make_engine(name, "float32", random_seed=2).generate(input_ids=prompts, sampling_params=sps)
    assert [o["token_ids"] for o in other] != [o["token_ids"] for o in a]
    greedy = make_engine(name, "float32").generate(input_ids=prompts[0], sampling_params={"max_new_tokens": 6, "ignore_eos": True})
    assert greedy["token_ids"] == P.greedy_generate(cfg, weights(name), prompts[0], 6, device="cpu")


def test_stream_and_eos_stop():
    name, cfg = "A", CONFIGS["A"]
    eng = make_engine(name, "float32")
    p = random_tokens(9, cfg["vocab_size"], 1300)
    want = P.greedy_generate(cfg, weights(name), p, 5, device="cpu")
    chunks = list(eng.generate(input_ids=p, sampling_params={"max_new_tokens": 5, "ignore_eos": True}, stream=True))
    assert [len(c["token_ids"]) for c in chunks] == [1, 2, 3, 4, 5] and chunks[-1]["token_ids"] == want
    k = max(i for i in range(5) if want[i] not in want[:i])          # generation stops at the first occurrence
    out = eng.generate(input_ids=p, sampling_params={"max_new_tokens": 5, "eos_token_id": want[k]})
    assert out["token_ids"] == want[:k + 1] and out["meta_info"]["finish_reason"] == {"type": "stop", "matched": want[k]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlapped_decode_gives_the_same_tokens(dtype):
    """The engine launches a decode step before it has read the tokens of the step before (they are put in
    place on the device).  Same tokens, stop tokens and counts as with every step read first."""
    name, cfg = "B", CONFIGS["B"]
    prompts = [random_tokens(n, cfg["vocab_size"], 1400 + n) for n in (7, 16, 23, 31, 5)]
    greedy = {"temperature": 0.0, "max_new_tokens": 14, "ignore_eos": True}
    a = make_engine(name, dtype, disable_overlap=True)
    b = make_engine(name, dtype)
    assert not a.scheduler.lookahead and b.scheduler.lookahead
    base = a.generate(input_ids=prompts, sampling_params=greedy)
    steps_before = b.scheduler.stats["steps"]
    look = b.generate(input_ids=prompts, sampling_params=greedy)
    assert [o["token_ids"] for o in look] == [o["token_ids"] for o in base]
    assert b.scheduler.stats["steps"] - steps_before == a.scheduler.stats["steps"]
    # stop tokens are seen one step late: the extra step's result must not leak into the output
    stop = base[1]["token_ids"][4]
    sps = [{"temperature": 0.0, "max_new_tokens": 3 + 2 * i, "eos_token_id": stop} for i in range(5)]
    base = a.generate(input_ids=prompts, sampling_params=sps)
    look = b.generate(input_ids=prompts, sampling_params=sps)
    assert [(o["token_ids"], o["meta_info"]["finish_reason"]) for o in look] == \
           [(o["token_ids"], o["meta_info"]["finish_reason"]) for o in base]
    assert any(o["meta_info"]["finish_reason"]["type"] == "stop" for o in base)
    # sampling with temperature draws the same numbers
    sps = [{"temperature": 0.8, "max_new_tokens": 9, "ignore_eos": True, "seed": 5 + i} for i in range(5)]
    assert [o["token_ids"] for o in b.generate(input_ids=prompts, sampling_params=sps)] == \
           [o["token_ids"] for o in a.generate(input_ids=prompts, sampling_params=sps)]
    # requests that arrive while others decode
    r1 = b.add_request(input_ids=prompts[0], sampling_params=greedy)
    for _ in range(4):
        b.step()
    r2 = b.add_request(input_ids=prompts[3], sampling_params=greedy)
    while not (r1.finished and r2.finished):
        b.step()
    want = a.generate(input_ids=[prompts[0], prompts[3]], sampling_params=greedy)
    assert [r1.output, r2.output] == [o["token_ids"] for o in want]
    while not b.scheduler.idle:
        b.step()
    a.scheduler.check_idle_invariants()
    b.scheduler.check_idle_invariants()


def test_command_line():
    name, cfg = "A", CONFIGS["A"]
    p = random_tokens(6, cfg["vocab_size"], 1400)
    proc = subprocess.run([sys.executable, "-m", "mini_sglang_b200.engine.cli", "--model", model_dir(name), "--dtype", "float32",
                           "--page_size", "1", "--num_pages", "64", "--max_num_reqs", "4", "--log_level", "ERROR",
                           "--input_ids", ",".join(map(str, p)), "--max_new_tokens", "4", "--ignore_eos"],
                          capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    out = json.loads(proc.stdout.strip().split("\n")[-1])
    assert out["token_ids"] == P.greedy_generate(cfg, weights(name), p, 4, device="cpu")


def test_dummy_load_runs_without_a_checkpoint(tmp_path):
    from mini_sglang_b200 import Engine, EngineArgs
    with open(tmp_path / "config.json", "w") as f:
        json.dump(CONFIGS["C"], f)
    eng = Engine(EngineArgs(model=str(tmp_path), dummy_load=True, random_seed=3, page_size=16, num_pages=16,
                            max_num_reqs=2, log_level="ERROR"))
    out = eng.generate(input_ids=[1, 2, 3], sampling_params={"max_new_tokens": 3, "ignore_eos": True})
    assert len(out["token_ids"]) == 3


def test_missing_extension_or_cpu_tensor_fails_loudly():
    from mini_sglang_b200 import ops
    with pytest.raises(ops.KernelError, match="CUDA device only"):
        ops.swiglu(torch.zeros(2, 8))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_portions_are_shared_while_the_first_prompt_is_still_fed(dtype):
    """Prompts go in 16 tokens a step.  Two requests share 64 tokens; the second is let in as soon as the first
    one's shared pages are in the prefix cache (well before the first prompt is done), takes all 64 tokens from
    there, and generates what the plain implementation generates."""
    name, cfg = "B", CONFIGS["B"]
    shared = random_tokens(64, cfg["vocab_size"], 1500)
    first = shared + random_tokens(70, cfg["vocab_size"], 1501)
    second = shared + random_tokens(9, cfg["vocab_size"], 1502)
    eng = make_engine(name, dtype, chunk_size=16, max_prefill_tokens=64)
    sp = {"max_new_tokens": 5, "ignore_eos": True}
    r1 = eng.add_request(input_ids=first, sampling_params=sp)
    r2 = eng.add_request(input_ids=second, sampling_params=sp)
    started = None
    for step in range(100):
        if r1.finished and r2.finished:
            break
        eng.step()
        if started is None and r2.slot is not None:
            started = step
            assert not r1.output                          # the first request has not produced a token yet
    assert started == 4 and r2.cached_tokens == 64 and r1.cached_tokens == 0
    while not eng.scheduler.idle:
        eng.step()
    if dtype == "float32":
        assert r1.output == P.greedy_generate(cfg, weights(name), first, 5, device="cpu")
        assert r2.output == P.greedy_generate(cfg, weights(name), second, 5, device="cpu")
    else:
        for prompt, r in ((first, r1), (second, r2)):
            ref = plain_logits(name, prompt + r.output)
            for i, t in enumerate(r.output):
                row = ref[len(prompt) - 1 + i]
                assert row[t] >= row.max() - 0.02, (i, t, row[t].item(), row.max().item())
    eng.scheduler.check_idle_invariants()


def test_profile_records_log_lines_and_async_generate(tmp_path, caplog):
    """--profile: one record per step with what it held and its times, saved as JSON; INFO log lines for steps
    with prompt tokens and for every 64th step without; `async_generate` from several coroutines at once."""
    import asyncio
    import logging
    name, cfg = "A", CONFIGS["A"]
    eng = make_engine(name, "float32", profile=True, profile_dir=str(tmp_path), log_level="INFO")
    prompts = [random_tokens(n, cfg["vocab_size"], 1600 + n) for n in (5, 9, 13)]
    sp = {"max_new_tokens": 70, "ignore_eos": True}
    with caplog.at_level(logging.INFO, logger="mini_sglang_b200.scheduler"):
        outs = eng.generate(input_ids=prompts, sampling_params=sp)
    assert [len(o["token_ids"]) for o in outs] == [70] * 3
    lines = [r.getMessage() for r in caplog.records]
    assert any(l.startswith("Extend #BS: 3  #Tokens: 27  #PrefixTokens: 0  #ExtendTokens: 27") for l in lines), lines
    decode_lines = [l for l in lines if l.startswith("Decode #BS: 3")]
    assert len(decode_lines) == 2 and "#CUDA-Graph: True" in decode_lines[0] and "#new-token-ratio" in decode_lines[0]
    recs = eng.step_records
    assert recs[0]["kind"] == "extend" and recs[0]["prompt_tokens"] == 27 and recs[0]["batch"] == 3
    assert all(r["kind"] == "decode" and r["tokens"] == 3 and r["cuda_graph"] for r in recs[1:])
    assert len(recs) == 70 and all(r["device_ms"] > 0 and r["kernels"] > 0 and r["host_ms"] > 0 for r in recs)
    path = eng.write_profile()
    saved = json.load(open(path))
    assert saved["summary"]["decode"]["steps"] == 69 and saved["summary"]["extend"]["tokens"] == 27
    assert len(saved["steps"]) == 70 and eng.write_profile() is None          # nothing new to save

    async def many():
        a = eng.async_generate(input_ids=prompts[0], sampling_params={"max_new_tokens": 6, "ignore_eos": True})
        b = eng.async_generate(input_ids=prompts[1], sampling_params={"max_new_tokens": 4, "ignore_eos": True})

        async def streamed():
            got = []
            async for part in await eng.async_generate(input_ids=prompts[2], stream=True,
                                                       sampling_params={"max_new_tokens": 5, "ignore_eos": True}):
                got.append(list(part["token_ids"]))
            return got
        return await asyncio.gather(a, b, streamed())

    ra, rb, rc = asyncio.run(many())
    assert ra["token_ids"] == outs[0]["token_ids"][:6] and rb["token_ids"] == outs[1]["token_ids"][:4]
    assert rc[-1] == outs[2]["token_ids"][:5] and [len(x) for x in rc] == sorted({len(x) for x in rc})
    while not eng.scheduler.idle:
        eng.step()
    eng.scheduler.check_idle_invariants()
    from mini_sglang_b200.parts import model as _model
    _model.NVTX_RANGES = False


def _folder_with_a_tokenizer(tmp_path, name):
    """A copy of a tiny model's folder with a word-level tokenizer beside it: the word "w<i>" is token i."""
    import shutil

    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import WhitespaceSplit
    d = str(tmp_path / "model")
    shutil.copytree(model_dir(name), d)
    tok = Tokenizer(WordLevel({f"w{i}": i for i in range(CONFIGS[name]["vocab_size"])}, unk_token="w0"))
    tok.pre_tokenizer = WhitespaceSplit()
    tok.save(os.path.join(d, "tokenizer.json"))
    with open(os.path.join(d, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast"}, f)
    return d


def test_text_prompts_through_the_entry_point_and_the_command_line(tmp_path):
    """With a tokenizer in the model folder a prompt may be text: it is encoded on the way in and the new tokens are
    decoded on the way out; the tokens are those of the same request given as ids, a list of texts runs as a batch, and
    the command line takes --prompt and lines of text in --prompt_file.  Without a tokenizer a text prompt is refused."""
    from mini_sglang_b200 import Engine, EngineArgs
    name, cfg = "A", CONFIGS["A"]
    d = _folder_with_a_tokenizer(tmp_path, name)
    ids = random_tokens(7, cfg["vocab_size"], 1700)
    other = random_tokens(4, cfg["vocab_size"], 1701)
    text, other_text = " ".join(f"w{t}" for t in ids), " ".join(f"w{t}" for t in other)
    sp = {"max_new_tokens": 5, "ignore_eos": True}
    want = P.greedy_generate(cfg, weights(name), ids, 5, device="cpu")
    want_other = P.greedy_generate(cfg, weights(name), other, 5, device="cpu")
    eng = Engine(EngineArgs(model=d, dtype="float32", page_size=PAGE[name], num_pages=128, max_num_reqs=4, random_seed=0,
                            log_level="ERROR"))
    out = eng.generate(prompt=text, sampling_params=sp)
    assert out["token_ids"] == want and out["text"] == " ".join(f"w{t}" for t in want) and out["meta_info"]["prompt_tokens"] == 7
    both = eng.generate(prompt=[other_text, text], sampling_params=sp)
    assert [o["token_ids"] for o in both] == [want_other, want]
    last = None
    for last in eng.generate(prompt=text, sampling_params=sp, stream=True):
        pass
    assert last["token_ids"] == want and last["text"].split() == [f"w{t}" for t in want]
    plain_eng = make_engine(name, "float32")
    with pytest.raises(ValueError, match="no tokenizer"):
        plain_eng.generate(prompt=text, sampling_params=sp)
    lines = tmp_path / "prompts.txt"
    lines.write_text(other_text + "\n" + json.dumps(ids) + "\n")
    proc = subprocess.run([sys.executable, "-m", "mini_sglang_b200.engine.cli", "--model", d, "--dtype", "float32",
                           "--page_size", "1", "--num_pages", "128", "--max_num_reqs", "4", "--log_level", "ERROR",
                           "--prompt", text, "--prompt_file", str(lines), "--max_new_tokens", "5", "--ignore_eos"],
                          capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    outs = [json.loads(l) for l in proc.stdout.strip().split("\n")[-3:]]
    assert [o["token_ids"] for o in outs] == [want, want_other, want]
    assert outs[0]["text"] == " ".join(f"w{t}" for t in want)


def test_long_prompts_under_a_small_pool_twice_the_same(tmp_path):
    """Forty requests with prompts of 20...4,000 tokens (a third of them behind a shared prefix of 400) and 20...90 new tokens
    each, through the scheduler with 16 slots, portions of 512 tokens and a pool that holds a fraction of them (requests wait,
    are retracted and come back; decode steps take the even cut of the keys or the cut per request as the lengths ask).  In
    bfloat16 two runs give the same tokens, request by request; the float32 run of the same requests gives the same first
    five tokens everywhere (later ones may part by rounding); nothing is left allocated."""
    from mini_sglang_b200 import Engine, EngineArgs
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 128,
           "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 192, "vocab_size": 503,
           "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192,
           "hidden_act": "silu", "attention_bias": False, "torch_dtype": "bfloat16"}
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    g = torch.Generator().manual_seed(4)
    draw = lambda lo, hi: int(torch.randint(lo, hi, (1,), generator=g))       # noqa: E731
    shared = torch.randint(0, 503, (400,), generator=g).tolist()
    prompts, params = [], []
    for i in range(40):
        n = draw(20, 300) if draw(0, 2) else draw(900, 4000)
        body = torch.randint(0, 503, (n,), generator=g).tolist()
        prompts.append(shared + body if i % 3 == 0 else body)
        params.append({"temperature": 0.0, "max_new_tokens": draw(20, 90), "ignore_eos": True})

    def run(dtype):
        eng = Engine(EngineArgs(model=str(tmp_path), dummy_load=True, random_seed=1, dtype=dtype, page_size=16, num_pages=700,
                                max_num_reqs=16, max_prefill_tokens=2048, chunk_size=512, log_level="ERROR", max_context_len=6000))
        outs = eng.generate(input_ids=prompts, sampling_params=params)
        eng.scheduler.check_idle_invariants()
        return [o["token_ids"] for o in outs], [o["meta_info"]["cached_tokens"] for o in outs], dict(eng.scheduler.stats)

    a, cached, stats = run("bfloat16")
    b, _, _ = run("bfloat16")
    assert a == b
    assert stats["retractions"] + stats.get("evicted_pages", 0) > 0, stats          # the pool was too small for what was live
    assert [len(x) for x in a] == [p["max_new_tokens"] for p in params]
    assert sum(1 for c in cached if c >= 400 - 16) >= 5          # the shared prefix came from the cache for most who have it
    f, _, _ = run("float32")
    assert [x[:5] for x in a] == [y[:5] for y in f]


def test_temperature_sampling_does_not_depend_on_the_pool_or_on_other_engines():
    """A request's random draws are keyed by the engine's seed, the request's number among those given to its engine and
    the step.  So a second engine in the same process with the same seed gives the same tokens, and so does one whose pool is
    so small that a request is retracted and fed again, with the overlapped decode or without.  float32."""
    from mini_sglang_b200 import Engine, EngineArgs
    name, cfg = "B", CONFIGS["B"]
    prompts = [random_tokens(n, cfg["vocab_size"], 4000 + i) for i, n in enumerate([30, 9, 55, 17, 41, 23, 60, 12, 35, 48])]
    sps = [{"temperature": 0.8, "max_new_tokens": 40, "ignore_eos": True} for _ in prompts]

    def run(pages, **kw):
        eng = Engine(EngineArgs(model=model_dir(name), dtype="float32", page_size=PAGE[name], num_pages=pages, max_num_reqs=8,
                                random_seed=5, log_level="ERROR", **kw))
        outs = eng.generate(input_ids=prompts, sampling_params=sps)
        eng.scheduler.check_idle_invariants()
        return [o["token_ids"] for o in outs], eng.scheduler.stats["retractions"]

    roomy, r0 = run(400)
    again, _ = run(400)
    tight, r1 = run(60)
    tight_no_overlap, r2 = run(60, disable_overlap=True)
    assert r0 == 0 and r1 > 0 and r2 > 0
    assert roomy == again == tight == tight_no_overlap
    assert len({tuple(t) for t in roomy}) == len(roomy)              # and the requests do not all draw alike


def test_edges_of_the_entry_point():
    """More requests than the largest captured batch; the context's end; a prompt that does not fit; requests aborted while
    others run; a one-token prompt; and what is refused before it reaches a step (no prompt, no new tokens, a token id outside
    the vocabulary), after which the engine goes on as before.  float32, greedy, against the plain implementation."""
    from mini_sglang_b200 import Engine, EngineArgs
    name, cfg = "B", CONFIGS["B"]
    prompts = [random_tokens(n, cfg["vocab_size"], 5000 + i) for i, n in enumerate([30, 9, 55, 17, 41])]
    plain = lambda p, n: P.greedy_generate(cfg, weights(name), p, n, device="cpu")      # noqa: E731
    sp = {"max_new_tokens": 12, "ignore_eos": True}
    eng = make_engine(name, "float32", max_capture_bs=2)
    assert [o["token_ids"] for o in eng.generate(input_ids=prompts, sampling_params=sp)] == [plain(p, 12) for p in prompts]

    eng = make_engine(name, "float32", max_context_len=40)
    out = eng.generate(input_ids=prompts[0], sampling_params={"max_new_tokens": 100, "ignore_eos": True})
    assert out["meta_info"]["finish_reason"] == {"type": "length", "length": 11} and out["token_ids"] == plain(prompts[0], 11)
    out = eng.generate(input_ids=prompts[2], sampling_params=sp)
    assert out["meta_info"]["finish_reason"]["type"] == "abort" and "does not fit" in out["meta_info"]["finish_reason"]["message"]
    assert out["token_ids"] == []

    eng = make_engine(name, "float32")
    reqs = [eng.add_request(input_ids=p, sampling_params={"max_new_tokens": 30, "ignore_eos": True}) for p in prompts]
    for _ in range(6):
        eng.step()
    eng.scheduler.abort(reqs[1].rid)
    eng.scheduler.abort(reqs[3].rid)
    while not eng.scheduler.idle:
        eng.step()
    eng.scheduler.check_idle_invariants()
    assert [r.finish_reason.to_json()["type"] for r in reqs] == ["length", "abort", "length", "abort", "length"]
    assert all(len(reqs[i].output) == 30 for i in (0, 2, 4)) and all(0 < len(reqs[i].output) < 30 for i in (1, 3))
    assert all(r.output == plain(p, len(r.output)) for r, p in zip(reqs, prompts))

    assert eng.generate(input_ids=[7], sampling_params={"max_new_tokens": 1, "ignore_eos": True})["token_ids"] == plain([7], 1)
    for bad, words in [(dict(input_ids=[7], sampling_params={"max_new_tokens": 0}), "max_new_tokens"),
                       (dict(input_ids=[], sampling_params=sp), "at least one prompt token"),
                       (dict(input_ids=[3, cfg["vocab_size"] + 5], sampling_params=sp), "vocabulary"),
                       (dict(input_ids=[-1], sampling_params=sp), "vocabulary"),
                       (dict(sampling_params=sp), "prompt or input_ids")]:
        with pytest.raises(ValueError, match=words):
            eng.generate(**bad)
    assert eng.scheduler.idle
    assert eng.generate(input_ids=prompts[1], sampling_params=sp)["token_ids"] == plain(prompts[1], 12)
    eng.scheduler.check_idle_invariants()
