"""The engine against the plain implementation, in float32 and bfloat16, at the tiny
configurations: every way of cutting the work must give the same logits at a position."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import PAGE, check_against_plain, make_runner, model_dir, plain_logits, play
from tiny_models import CONFIGS, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C"]


def seqs_for(name, lens, base=100):
    V = CONFIGS[name]["vocab_size"]
    return {f"r{i}": random_tokens(n, V, base + i) for i, n in enumerate(lens)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_alone(name, dtype):
    seqs = seqs_for(name, [5, 9, 13, 70])
    runner = make_runner(name, dtype, num_pages=256)
    steps = [{"entries": [(rid, toks, list(range(len(toks))))], "end": [rid]} for rid, toks in seqs.items()]
    got = play(runner, steps)
    assert len(got) == sum(len(t) for t in seqs.values())
    check_against_plain(name, dtype, got, seqs)
    runner.mgr.check_idle()


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_bulk_then_last_32_one_by_one(name, dtype, graphs):
    seqs = seqs_for(name, [80], base=200)
    toks = seqs["r0"]
    runner = make_runner(name, dtype, num_pages=256, graphs=graphs)
    n0 = len(toks) - 32
    steps = [{"entries": [("r0", toks[:n0], [n0 - 1])]}]
    steps += [{"entries": [("r0", [toks[i]], [0])]} for i in range(n0, len(toks))]
    got = play(runner, steps)
    assert len(got) == 33
    check_against_plain(name, dtype, got, seqs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_changing_size(name, dtype):
    seqs = seqs_for(name, [97], base=300)
    toks = seqs["r0"]
    sizes, i = [], 0
    pattern = [7, 2, 5, 3, 2, 16, 2, 1, 9, 31, 2, 4]
    while sum(sizes) < len(toks):
        sizes.append(min(pattern[i % len(pattern)], len(toks) - sum(sizes)))
        i += 1
    runner = make_runner(name, dtype, num_pages=256)
    steps, p = [], 0
    for n in sizes:
        steps.append({"entries": [("r0", toks[p:p + n], list(range(n)))]})
        p += n
    got = play(runner, steps)
    assert len(got) == len(toks)
    check_against_plain(name, dtype, got, seqs)


def mixed_trace(seqs):
    """Up to four live requests; portions of some beside decoded tokens of others; requests end and
    new ones start so that their pages are handed out again."""
    order = list(seqs)
    pos = {r: 0 for r in order}
    live, waiting, steps = [], list(order), []
    chunk_cycle = [6, 2, 11, 3]
    k = 0
    while live or waiting:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        entries, end = [], []
        for j, r in enumerate(list(live)):
            toks = seqs[r]
            bulk = len(toks) - 8                       # the last 8 tokens go one by one
            if pos[r] < bulk:
                n = min(chunk_cycle[(k + j) % 4], bulk - pos[r])
            else:
                n = 1
            if (k + j) % 5 == 4 and len(live) > 1:
                continue                               # left out of this step, goes on later
            want = [n - 1] if n > 1 else [0]
            entries.append((r, toks[pos[r]:pos[r] + n], want))
            pos[r] += n
            if pos[r] == len(toks):
                end.append(r)
                live.remove(r)
        if entries:
            steps.append({"entries": entries, "end": end})
        k += 1
    return steps


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_with_page_reuse(name, dtype):
    lens = [23, 40, 17, 31, 52, 19, 44, 28]
    seqs = seqs_for(name, lens, base=400)
    P = PAGE[name]
    # room for the four largest at once, rounded up to pages, and no more: pages are reused
    need = sum(sorted(-(-n // P) for n in lens)[-4:])
    runner = make_runner(name, dtype, num_pages=need)
    steps = mixed_trace(seqs)
    # poison whatever is not in use: stale or foreign pages must never be read
    for k, v in runner.storage.kv.values():
        k.fill_(float("nan"))
        v.fill_(float("nan"))
        k[0].zero_()
        v[0].zero_()
    got = play(runner, steps)
    check_against_plain(name, dtype, got, seqs)
    runner.mgr.check_idle()
    assert runner.mgr.groups[0].pool.available == need


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    name = "B"
    seqs = seqs_for(name, [300], base=500)
    toks = seqs["r0"]
    runner = make_runner(name, dtype, num_pages=128)
    steps = [{"entries": [("r0", toks[:4], [3])]}]
    steps += [{"entries": [("r0", [toks[i]], [0])]} for i in range(4, len(toks))]
    got = play(runner, steps)
    check_against_plain(name, dtype, got, seqs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens(name, dtype):
    seqs = seqs_for(name, [6, 1, 2], base=600)
    runner = make_runner(name, dtype, num_pages=64)
    steps = [{"entries": [("r0", [seqs["r0"][i]], [0])]} for i in range(6)]
    steps += [{"entries": [("r1", seqs["r1"], [0]), ("r2", seqs["r2"], [0, 1])]}]
    got = play(runner, steps)
    check_against_plain(name, dtype, got, seqs)


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_key_matters(dtype):
    """Make one far key decisive: scale q_norm/k_norm-free inputs is not possible from outside, so
    use a prompt whose first token repeats at the end; then check that cutting the cache at a page
    edge (page size 16, key tile 64) does not change the answer at position 200."""
    name = "C"
    seqs = seqs_for(name, [201], base=700)
    toks = seqs["r0"]
    runner = make_runner(name, dtype, num_pages=64)
    got = play(runner, [{"entries": [("r0", toks[:64], [])]}, {"entries": [("r0", toks[64:128], [])]},
                        {"entries": [("r0", toks[128:200], [])]}, {"entries": [("r0", toks[200:], [0])]}])
    check_against_plain(name, dtype, got, seqs)


def test_trace_run_program(tmp_path):
    name = "B"
    seqs = seqs_for(name, [37, 21], base=800)
    a, b = seqs["r0"], seqs["r1"]
    lines = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [0, 19]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[20:35], "want": []}, {"id": "b", "tokens": b[:21], "want": [20]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[35:37], "want": [0, 1]}], "end": ["a"]},
    ]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir(name),
                               "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                              input="\n".join(json.dumps(l) for l in lines) + "\n", capture_output=True, text=True,
                              timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        V = CONFIGS[name]["vocab_size"]
        ra, rb = plain_logits(name, a), plain_logits(name, b)
        s0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V))
        s1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V))
        s2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V))
        from helpers import assert_rows_close
        assert_rows_close(s0, ra[[0, 19]], dtype)
        assert_rows_close(s1, rb[[20]], dtype)
        assert_rows_close(s2, ra[[35, 36]], dtype)


def test_step_fields_made_on_the_device_equal_the_hosts(monkeypatch):
    """Decode steps through a CUDA graph get their fields (positions, lengths, cache slots, block-table rows, kv splits) from
    a kernel that reads a device copy of the block tables, kept up to date by deltas.  Requests come, grow over page edges,
    end and are replaced, with so few pages that they are used again; before every replay the graph's buffer must hold
    exactly what the host's own filling of the same step gives."""
    from mini_sglang_b200 import ops
    from mini_sglang_b200.engine.step import StepEntry
    name = "B"
    cfg = CONFIGS[name]
    runner = make_runner(name, "bfloat16", num_pages=40, max_reqs=6, page_size=4)
    assert runner.device_meta and runner.use_cuda_graph
    checked = []
    inner = runner._meta_on_device

    def checking(gr, entries, starts, nsplits, b, even_cuts=None):
        inner(gr, entries, starts, nsplits, b, even_cuts)
        lay = gr.layout
        want = np.zeros(lay.size, dtype=np.int32)
        runner._fill(want, lay, entries, starts, list(range(b)), nsplits, pad_to=b, even_cuts=even_cuts)
        got = gr.dev.cpu().numpy()
        B = len(entries)
        for field, off, n in [("input_ids", lay.input_ids, b), ("positions", lay.positions, b), ("token_req", lay.token_req, b),
                              ("q_start", lay.q_start, b + 1), ("kv_len", lay.kv_len, b), ("slots", lay.slots, b), ("want", lay.want, b)]:
            assert (got[off:off + n] == want[off:off + n]).all(), (field, got[off:off + n], want[off:off + n])
        for gi, g in enumerate(runner.mgr.groups):
            mp = lay.max_pages[gi]
            assert (got[lay.out_loc[gi]: lay.out_loc[gi] + b] == want[lay.out_loc[gi]: lay.out_loc[gi] + b]).all()
            assert (got[lay.nsplit[gi]: lay.nsplit[gi] + b] == want[lay.nsplit[gi]: lay.nsplit[gi] + b]).all()
            order = got[lay.order[gi]: lay.order[gi] + b]
            assert (order == want[lay.order[gi]: lay.order[gi] + b]).all(), (order, want[lay.order[gi]: lay.order[gi] + b])
            assert sorted(order.tolist()) == list(range(b))
            n_even = ops.even_cut_size(b, lay.even_nb[gi]) if lay.even_nb[gi] else 0
            assert (got[lay.even[gi]: lay.even[gi] + n_even] == want[lay.even[gi]: lay.even[gi] + n_even]).all()
            tg, tw = got[lay.table[gi]: lay.table[gi] + b * mp].reshape(b, mp), want[lay.table[gi]: lay.table[gi] + b * mp].reshape(b, mp)
            for r, e in enumerate(entries):                 # the pages a request holds; what lies beyond them is never read
                n = int(g.n_pages[e.slot])
                assert (tg[r, :n] == tw[r, :n]).all(), (r, tg[r, :n], tw[r, :n])
            assert (tg[B:] == 0).all()
        checked.append(b)

    monkeypatch.setattr(runner, "_meta_on_device", checking)
    rnd = np.random.RandomState(0)
    live = {}
    for it in range(60):
        if len(live) < 5 and (not live or rnd.rand() < 0.4):
            s = runner.open()
            n = int(rnd.randint(1, 14))
            runner.step([StepEntry(s, random_tokens(n, cfg["vocab_size"], 3000 + it), [])])
            live[s] = n
        if live and rnd.rand() < 0.15:
            s = list(live)[int(rnd.randint(len(live)))]
            runner.close(s)
            del live[s]
        some = [s for s in live if rnd.rand() < 0.8 and live[s] < 30]
        if some:
            out = runner.step([StepEntry(s, [int(rnd.randint(cfg["vocab_size"]))], [0]) for s in some])
            assert out.shape[0] == len(some) and torch.isfinite(out).all()
            for s in some:
                live[s] += 1
    assert len(checked) > 25 and len(set(checked)) >= 3
    for s in live:
        runner.close(s)


@pytest.mark.parametrize("fields_on_device", [True, False])
def test_even_cut_of_requests_of_mixed_lengths(monkeypatch, fields_on_device):
    """Decode steps whose requests hold 1,030 to 3,000 keys: the keys of all of them are dealt out evenly over the blocks
    that the SMs hold (a block takes the end of one request and the start of the next; a request is merged from up to
    48 pieces).  Requests end and others join, pages are used again, the fields of every step are made on the device and
    compared with the host's (or, second run, written by the host and copied).  bfloat16, two layers of a small width,
    every decoded row against the plain implementation."""
    import plain_qwen3 as P
    from helpers import assert_row_close
    from mini_sglang_b200 import ops
    from mini_sglang_b200.config import Qwen3Config
    from mini_sglang_b200.config.qwen3 import build_qwen3_spec
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    from mini_sglang_b200.parts import expected_tensors
    from mini_sglang_b200.weights import RandomSource
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 96,
           "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 160, "vocab_size": 411,
           "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 4096,
           "hidden_act": "silu", "attention_bias": False, "torch_dtype": "bfloat16"}
    spec = build_qwen3_spec(Qwen3Config.from_dict(cfg))
    src = RandomSource(expected_tensors(spec), 5, torch.bfloat16, "cuda")
    weights = {n: src.draw(n) for n in expected_tensors(spec) if src.has(n)}
    lens = {"a": 1100, "b": 2300, "c": 3000, "d": 1500, "e": 1030, "f": 2048}
    n_dec = 6
    seqs = {r: random_tokens(n + n_dec, cfg["vocab_size"], 900 + i) for i, (r, n) in enumerate(lens.items())}
    pages = sum(-(-(lens[r] + n_dec) // 16) for r in "abcd") + 2          # room for four of them at a time
    runner = ModelRunner.from_random(spec, 5, dtype="bfloat16", page_size=16, num_pages=pages, max_reqs=4)
    assert runner.device_meta and runner._even_nb
    slots, fed, got, plans = {}, {}, {}, []
    inner = runner._meta_on_device

    def checking(gr, entries, starts, nsplits, b, even_cuts=None):
        inner(gr, entries, starts, nsplits, b, even_cuts)
        lay = gr.layout
        want = np.zeros(lay.size, dtype=np.int32)
        runner._fill(want, lay, entries, starts, list(range(b)), nsplits, pad_to=b, even_cuts=even_cuts)
        have = gr.dev.cpu().numpy()
        n_even = ops.even_cut_size(b, lay.even_nb[0])
        for off, n in [(lay.even[0], n_even), (lay.nsplit[0], b), (lay.kv_len, b), (lay.out_loc[0], b)]:
            assert (have[off:off + n] == want[off:off + n]).all(), (have[off:off + n], want[off:off + n])

    if fields_on_device:
        monkeypatch.setattr(runner, "_meta_on_device", checking)
    else:
        runner.device_meta = False              # the host writes every field of the step and copies them (the other way to a replay)

    def feed(r):
        slots[r], fed[r] = runner.open(), lens[r]
        runner.step([StepEntry(slots[r], seqs[r][:lens[r]], [])])

    def decode(rs):
        out = runner.step([StepEntry(slots[r], [seqs[r][fed[r]]], [0]) for r in rs]).float().cpu()
        assert runner.last_step_used_graph and runner.last_plan["graph_key"][2] == "even", runner.last_plan
        plans.append(runner.last_plan)
        for r, row in zip(rs, out):
            got[(r, fed[r])] = row
            fed[r] += 1

    for r in "abcd":
        feed(r)
    decode("abcd")
    decode("abcd")
    runner.close(slots.pop("b"))
    decode("acd")
    feed("e")                                   # takes pages that b held
    decode("acde")
    runner.close(slots.pop("c"))
    feed("f")
    decode("adef")
    decode("fa")
    assert max(max(p["nsplits"][0]) for p in plans) > 4 and min(min(p["nsplits"][0]) for p in plans) >= 1
    for r in lens:
        rows = sorted(pos for (rr, pos) in got if rr == r)
        with torch.no_grad():
            ref = P.forward_sequence(cfg, weights, seqs[r], device="cuda", rows=rows).cpu()
        for pos, want in zip(rows, ref):
            try:
                assert_row_close(got[(r, pos)], want, "bfloat16")
            except AssertionError as e:
                raise AssertionError(f"request {r}, position {pos}: {e}") from None


@pytest.mark.parametrize("head_dim,seed", [(64, 0), (128, 3)])
def test_random_requests_of_mixed_lengths_come_and_go(head_dim, seed):
    """A random run: up to 12 live requests, short prompts (20...300 tokens) beside long ones (900...5,000), requests join
    and leave at random, every step decodes one token of every live request through a CUDA graph (the even cut of the keys
    in most steps, the cut per request in the others).  bfloat16, two layers of a small width; every decoded row against the
    plain implementation."""
    import plain_qwen3 as P
    from helpers import assert_row_close
    from mini_sglang_b200.config import Qwen3Config
    from mini_sglang_b200.config.qwen3 import build_qwen3_spec
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    from mini_sglang_b200.parts import expected_tensors
    from mini_sglang_b200.weights import RandomSource
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 128,
           "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": head_dim, "intermediate_size": 192, "vocab_size": 503,
           "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192,
           "hidden_act": "silu", "attention_bias": False, "torch_dtype": "bfloat16"}
    spec = build_qwen3_spec(Qwen3Config.from_dict(cfg))
    src = RandomSource(expected_tensors(spec), 5, torch.bfloat16, "cuda")
    weights = {n: src.draw(n) for n in expected_tensors(spec) if src.has(n)}
    rnd = np.random.RandomState(seed)
    most, n_dec = 12, 60
    runner = ModelRunner.from_random(spec, 5, dtype="bfloat16", page_size=16, num_pages=most * 330 + 8, max_reqs=most)
    live, seqs, fed, got, modes = {}, {}, {}, {}, {}
    for it in range(n_dec):
        if len(live) < most and (len(live) < 3 or rnd.rand() < 0.3):
            n = int(rnd.choice([rnd.randint(20, 300), rnd.randint(900, 5000)]))
            rid = len(seqs)
            seqs[rid] = random_tokens(n + n_dec, cfg["vocab_size"], 7000 + 100 * seed + rid)
            live[rid], fed[rid] = runner.open(), n
            for i in range(0, n, 2048):
                runner.step([StepEntry(live[rid], seqs[rid][i:min(i + 2048, n)], [])])
        if live and rnd.rand() < 0.1:
            runner.close(live.pop(list(live)[rnd.randint(len(live))]))
        rs = list(live)
        if not rs:
            continue
        out = runner.step([StepEntry(live[r], [seqs[r][fed[r]]], [0]) for r in rs]).float().cpu()
        assert runner.last_step_used_graph
        mode = str(runner.last_plan["graph_key"][2])
        modes[mode] = modes.get(mode, 0) + 1
        for r, row in zip(rs, out):
            got[(r, fed[r])] = row
            fed[r] += 1
    assert modes.get("even", 0) >= n_dec // 3 and len(got) > 4 * n_dec, (modes, len(got))
    for rid in seqs:
        rows = sorted(p for (r, p) in got if r == rid)
        if not rows:
            continue
        with torch.no_grad():
            ref = P.forward_sequence(cfg, weights, seqs[rid][:rows[-1] + 1], device="cuda", rows=rows).cpu()
        for p, want in zip(rows, ref):
            try:
                assert_row_close(got[(rid, p)], want, "bfloat16")
            except AssertionError as e:
                raise AssertionError(f"head size {head_dim}, request {rid}, position {p}: {e}") from None
    for s in live.values():
        runner.close(s)
    runner.mgr.check_idle()
