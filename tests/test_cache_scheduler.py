"""Cache manager, prefix tree and scheduler on the CPU: no page lost, held twice or freed twice
under random orders of requests; what the scheduler decides when pages run out."""

import os
import random

import numpy as np
import pytest
import torch

from mini_sglang_b200.cache import CacheManager, OutOfPages, OutOfSlots, PagedKVNeed, PagePool, PrefixTree, StateNeed
from mini_sglang_b200.engine.scheduler import Req, Scheduler
from mini_sglang_b200.engine.step import StepEntry
from mini_sglang_b200.sampling import SamplingParams


# ---------------------------------------------------------------------------------------
def test_pool_fifo_and_double_free():
    pool = PagePool(5)
    a = pool.alloc(3)
    assert a == [1, 2, 3] and pool.available == 2
    pool.free([2])
    assert pool.alloc(3) == [4, 5, 2]              # first in, first out; page 0 never appears
    with pytest.raises(OutOfPages):
        pool.alloc(1)
    pool.free([1])
    with pytest.raises(ValueError, match="freed twice"):
        pool.free([1])
    with pytest.raises(ValueError):
        pool.free([0])


def all_held_pages(mgr, gi):
    g = mgr.groups[gi]
    out = []
    for slot in range(1, mgr.max_reqs + 1):
        if mgr.is_open(slot):
            out += [int(p) for p in g.table[slot, int(g.first_live[slot]):int(g.n_pages[slot])]]
    return out


@pytest.mark.parametrize("page_size", [1, 4, 16])
def test_manager_random_orders_no_page_lost_or_held_twice(page_size):
    rnd = random.Random(page_size)
    needs = {0: PagedKVNeed(2, 16), 1: PagedKVNeed(2, 16), 2: PagedKVNeed(1, 32, window=24), 3: StateNeed((4,))}
    mgr = CacheManager(needs, page_size=page_size, num_pages=400 // page_size, max_reqs=6, max_context_len=300,
                       max_step_tokens=40)
    assert len(mgr.groups) == 2 and mgr.groups[0].cache_ids == [0, 1] and mgr.groups[1].window == 24
    live = {}
    mirror = [np.zeros_like(g.table) for g in mgr.groups]
    for it in range(3000):
        op = rnd.random()
        if op < 0.25 and mgr.free_slots:
            live[mgr.open()] = 0
        elif op < 0.85 and live:
            slot = rnd.choice(list(live))
            n = rnd.choice([1, 1, 1, 2, 7, 33])
            if live[slot] + n > 300:
                continue
            try:
                mgr.reserve(slot, n)
            except OutOfPages:
                continue
            loc = mgr.slot_mapping(0, slot, live[slot], n)
            assert (loc >= page_size).all()                         # never the dump page
            mgr.commit(slot, n)
            live[slot] += n
        elif live:
            slot = rnd.choice(list(live))
            mgr.close(slot)
            del live[slot]
        for gi, g in enumerate(mgr.groups):
            held = all_held_pages(mgr, gi)
            assert len(held) == len(set(held)), "a page is held twice"
            assert 0 not in held
            assert len(held) + g.pool.available == g.pool.num_pages, "a page was lost"
            for slot, n_tok in live.items():
                # every token still inside the window has a live page
                lo = 0 if g.window is None else max(0, n_tok - g.window + 1)
                if n_tok:
                    pages = g.table[slot, lo // page_size: -(-n_tok // page_size)]
                    assert (pages > 0).all()
        # a copy of the block tables that only ever sees the rows reported as changed stays equal to them
        if it % 7 == 0:
            for gi, g in enumerate(mgr.groups):
                for slot, row in mgr.take_dirty_rows(gi):
                    mirror[gi][slot, :len(row)] = row
                assert not g.dirty
                for slot in live:
                    n = int(g.n_pages[slot])
                    assert (mirror[gi][slot, :n] == g.table[slot, :n]).all()
    for slot in list(live):
        mgr.close(slot)
    mgr.check_idle()
    with pytest.raises(ValueError, match="closed twice"):
        mgr.close(1)


def test_window_pages_are_given_back_as_the_window_passes():
    mgr = CacheManager({0: PagedKVNeed(1, 16, window=8)}, page_size=4, num_pages=6, max_reqs=2, max_context_len=1000,
                       max_step_tokens=4)
    s = mgr.open()
    total = mgr.groups[0].pool.num_pages
    for i in range(200):                      # far more tokens than the pool holds
        mgr.reserve(s, 1)
        mgr.commit(s, 1)
        assert mgr.groups[0].pool.in_use <= 4
    g = mgr.groups[0]
    assert g.first_live[s] == (200 - 8 + 1) // 4
    assert (g.table[s, :g.first_live[s]] == 0).all()
    mgr.close(s)
    assert g.pool.available == total


def test_slots_run_out_and_state_rows_are_zeroed():
    mgr = CacheManager({0: StateNeed((3,))}, page_size=4, num_pages=4, max_reqs=2, max_context_len=64)
    zeroed = []
    mgr.on_open.append(zeroed.append)
    a, b = mgr.open(), mgr.open()
    assert {a, b} == {1, 2} and zeroed == [a, b]
    with pytest.raises(OutOfSlots):
        mgr.open()
    mgr.close(a)
    assert mgr.open() == a


def test_reserve_is_all_or_nothing():
    mgr = CacheManager({0: PagedKVNeed(1, 16), 1: PagedKVNeed(1, 16, window=4)}, page_size=4, num_pages=5,
                       max_reqs=2, max_context_len=64, max_step_tokens=4)
    s = mgr.open()
    mgr.reserve(s, 16)
    before = [g.pool.available for g in mgr.groups]
    with pytest.raises(OutOfPages):
        mgr.reserve(s, 8)
    assert [g.pool.available for g in mgr.groups] == before and mgr.reserved[s] == 16


# ---------------------------------------------------------------------------------------
def test_prefix_tree_match_insert_lock_evict():
    P = 4
    tree = PrefixTree(P)
    toks = list(range(100, 119))                         # 19 tokens: 4 full pages
    table, dup, node = tree.insert(toks, [11, 12, 13, 14], owned_from=0)
    assert table == [11, 12, 13, 14] and dup == [] and tree.evictable_pages == 4
    pages, n2 = tree.match(toks[:-1])
    assert pages == [11, 12, 13, 14] and n2 is node
    pages, _ = tree.match(toks[:7])
    assert pages == [11]
    other = toks[:8] + [7, 7, 7, 7, 9]
    table, dup, node_b = tree.insert(other, [11, 12, 21], owned_from=2)
    assert table == [11, 12, 21] and dup == []
    # a request that computed the same content on pages of its own gets the tree's pages back
    table, dup, _ = tree.insert(toks, [31, 32, 33, 34], owned_from=0)
    assert table == [11, 12, 13, 14] and dup == [31, 32, 33, 34]
    tree.lock(node)
    assert tree.protected_pages == 4 and tree.evictable_pages == 1
    assert tree.evict(10) == [21]                        # only the unpinned leaf goes
    tree.unlock(node)
    assert tree.protected_pages == 0
    freed = tree.evict(10)
    assert sorted(freed) == [11, 12, 13, 14] and freed[0] == 14   # leaves first, parents follow
    assert tree.num_nodes == 0


def test_prefix_tree_lru_order():
    tree = PrefixTree(1)
    tree.insert([1, 2], [5, 6], 0)
    tree.insert([1, 3], [5, 7], 1)
    tree.match([1, 2])                                   # touch branch [1, 2]
    assert tree.evict(1) == [7]


# ---------------------------------------------------------------------------------------
class FakeRunner:
    """Keeps the real cache manager busy; the 'logits' at a wanted place depend only on the
    request's tokens up to that place, so any schedule must generate the same tokens.

    It also plays the cache itself: every page remembers which (position, token) was written into each of its
    places.  Before a request's tokens are 'computed', every earlier position that the request may still read
    must hold exactly that request's token in the page its block table names, so a page that two requests
    write, or a prefix page that was evicted and handed to someone else, fails the step that reads it."""

    V = 64

    def __init__(self, mgr):
        self.mgr = mgr
        self.history = {}
        self.steps = []
        self.lookahead_steps = 0
        self.content = [dict() for _ in mgr.groups]          # per group: page -> {place: (position, token)}

    supports_device_tokens = True

    def _check_owned_pages_are_private(self):
        for gi, g in enumerate(self.mgr.groups):
            seen = {}
            for slot in range(1, self.mgr.max_reqs + 1):
                if self.mgr.is_open(slot):
                    for p in self.mgr.owned_pages(slot, gi):
                        assert p not in seen, f"page {p} of group {gi} is owned by slots {seen[p]} and {slot}"
                        seen[p] = slot

    def step(self, entries, prev_ids=None):
        rows = []
        P = self.mgr.page_size
        self.steps.append([(e.slot, len(e.tokens)) for e in entries])
        self.lookahead_steps += prev_ids is not None
        short = [0] * len(self.mgr.groups)
        for e in entries:
            for gi, n in enumerate(self.mgr.pages_needed(e.slot, len(e.tokens))):
                short[gi] += n
        for gi, g in enumerate(self.mgr.groups):
            assert short[gi] <= g.pool.available, "the scheduler planned a step that does not fit"
        hists = []
        for e in entries:                                    # first every entry writes, as one batch does
            start = int(self.mgr.length[e.slot])
            # tokens before `start` may sit in pages taken over from the prefix cache: the request knows them
            req = next(r for r in self.sched.running if r.slot == e.slot)
            assert list(req.tokens[start:start + len(e.tokens)]) == list(e.tokens)
            fed = [int(prev_ids[-1 - t]) if t < 0 else t for t in e.tokens]      # -1 - r: row r of the tokens in flight
            hist = list(req.tokens[:start]) + fed
            assert min(hist) >= 0
            hists.append((start, hist))
            self.mgr.reserve(e.slot, len(e.tokens))
            for gi, g in enumerate(self.mgr.groups):
                for pos in range(start, start + len(e.tokens)):
                    page = int(g.table[e.slot, pos // P])
                    assert page > 0
                    self.content[gi].setdefault(page, {})[pos % P] = (pos, hist[pos])
        self._check_owned_pages_are_private()
        for e, (start, hist) in zip(entries, hists):         # then every entry reads
            end = start + len(e.tokens)
            for gi, g in enumerate(self.mgr.groups):
                lo = 0 if g.window is None else max(0, start - g.window + 1)
                for pos in range(lo, end):
                    page = int(g.table[e.slot, pos // P])
                    got = self.content[gi].get(page, {}).get(pos % P)
                    assert got == (pos, hist[pos]), \
                        f"slot {e.slot} reads position {pos} from page {page} of group {gi}: holds {got}, wants {(pos, hist[pos])}"
            for w in e.want:
                row = torch.zeros(self.V)
                row[hash(tuple(hist[:start + w + 1])) % (self.V - 1) + 1] = 1.0     # never token 0 (eos)
                rows.append(row)
            self.mgr.commit(e.slot, len(e.tokens))
        return torch.stack(rows) if rows else torch.zeros(0, self.V)


class ArgmaxSampler:
    def sample(self, logits, temperatures, row_keys, steps):
        return logits.argmax(-1)


def run_all(page_size, num_pages, prompts, max_new, *, chunk=8192, budget=16384, policy="lpm", max_reqs=8,
            prefix_cache=True, conservativeness=1.0, lookahead=False, ignore_eos=True, eos=0):
    mgr = CacheManager({0: PagedKVNeed(2, 16)}, page_size=page_size, num_pages=num_pages, max_reqs=max_reqs,
                       max_context_len=4096, max_step_tokens=budget)
    runner = FakeRunner(mgr)
    sch = Scheduler(runner, ArgmaxSampler(), max_num_reqs=max_reqs, max_step_tokens=budget, chunk_size=chunk,
                    policy=policy, enable_prefix_cache=prefix_cache, eos_ids=[eos], conservativeness=conservativeness,
                    retract_decode_steps=4, lookahead=lookahead)
    runner.sched = sch
    reqs = [Req(f"r{i}", p, SamplingParams(max_new_tokens=m, ignore_eos=ignore_eos)) for i, (p, m) in enumerate(zip(prompts, max_new))]
    for r in reqs:
        sch.add_request(r)
    guard = 0
    while not sch.idle:
        sch.step()
        guard += 1
        assert guard < 20000, "scheduler does not make progress"
    sch.check_idle_invariants()
    return reqs, sch, runner


def prompts_for(seed, n, lo, hi, shared=0):
    rnd = random.Random(seed)
    common = [rnd.randrange(1, 60) for _ in range(shared)]
    return [(common if (shared and i % 2 == 0) else []) + [rnd.randrange(1, 60) for _ in range(rnd.randrange(lo, hi))]
            for i in range(n)]


def test_scheduler_outputs_do_not_depend_on_the_schedule():
    prompts = prompts_for(1, 12, 5, 90, shared=40)
    max_new = [3 + (i * 7) % 20 for i in range(12)]
    base, sch0, _ = run_all(4, 4000, prompts, max_new, policy="fcfs", prefix_cache=False)
    want = [r.output for r in base]
    assert all(len(o) == m for o, m in zip(want, max_new))
    assert sch0.stats["retractions"] == 0
    for kw in [dict(page_size=1, num_pages=400), dict(page_size=16, num_pages=30, chunk=16, budget=48),
               dict(page_size=4, num_pages=70, chunk=7, budget=20, policy="lpm"),
               dict(page_size=4, num_pages=45, policy="random", max_reqs=3),
               dict(page_size=4, num_pages=60, policy="lof", prefix_cache=False)]:
        page_size, num_pages = kw.pop("page_size"), kw.pop("num_pages")
        reqs, sch, runner = run_all(page_size, num_pages, prompts, max_new, **kw)
        assert [r.output for r in reqs] == want, kw
        assert all(r.finish_reason.type == "length" for r in reqs)
        budget = kw.get("budget", 16384)
        assert all(sum(n for _, n in st) <= budget for st in runner.steps)
        assert all(n <= kw.get("chunk", 8192) for st in runner.steps for _, n in st)


def test_lookahead_decode_gives_the_same_tokens():
    """Launching the next decode step before the last tokens are read changes nothing but the timing:
    same outputs and finish reasons, with stop tokens (seen one step late), lengths, tiny pools."""
    prompts = prompts_for(3, 10, 5, 70, shared=36)
    max_new = [1 + (i * 5) % 17 for i in range(10)]
    for eos, ignore in [(0, True), (7, False), (23, False)]:
        for kw in [dict(page_size=4, num_pages=4000, policy="fcfs", prefix_cache=False),
                   dict(page_size=16, num_pages=30, chunk=16, budget=48),
                   dict(page_size=4, num_pages=45, policy="random", max_reqs=3),
                   dict(page_size=1, num_pages=300, policy="lpm")]:
            kw = dict(kw)
            page_size, num_pages = kw.pop("page_size"), kw.pop("num_pages")
            base, sch0, run0 = run_all(page_size, num_pages, prompts, max_new, eos=eos, ignore_eos=ignore, **kw)
            look, sch1, run1 = run_all(page_size, num_pages, prompts, max_new, eos=eos, ignore_eos=ignore, lookahead=True, **kw)
            assert run0.lookahead_steps == 0
            assert [r.output for r in look] == [r.output for r in base], (eos, kw)
            assert [r.finish_reason.type for r in look] == [r.finish_reason.type for r in base]
            assert all(t >= 0 for r in look for t in r.tokens)
    assert run1.lookahead_steps > 0
    stops = [r for r in look if r.finish_reason.type == "stop"]
    assert stops and all(r.tokens[-1] == 23 for r in stops)


def test_lookahead_with_requests_arriving_and_aborted_while_others_decode():
    """Random arrival times, lengths, stop tokens, aborts and pool sizes: the overlapped schedule gives every
    request the tokens and the finish reason of the read-first schedule, and leaves the cache idle."""
    rnd = random.Random(11)
    for trial in range(12):
        n = rnd.randrange(3, 9)
        prompts = prompts_for(100 + trial, n, 3, 60, shared=rnd.choice([0, 33]))
        max_new = [rnd.randrange(1, 25) for _ in range(n)]
        arrive = sorted(rnd.randrange(0, 30) for _ in range(n))
        abort_at = {rnd.randrange(n): rnd.randrange(5, 40)} if trial % 3 == 0 else {}
        page_size, num_pages = rnd.choice([(1, 400), (4, 60), (16, 24), (4, 4000)])
        eos, ignore = rnd.choice([(0, True), (7, False), (23, False)])
        results = []
        for lookahead in (False, True):
            mgr = CacheManager({0: PagedKVNeed(2, 16)}, page_size=page_size, num_pages=num_pages, max_reqs=4,
                               max_context_len=4096, max_step_tokens=64)
            runner = FakeRunner(mgr)
            sch = Scheduler(runner, ArgmaxSampler(), max_num_reqs=4, max_step_tokens=64, chunk_size=16, policy="fcfs",
                            eos_ids=[eos], retract_decode_steps=4, lookahead=lookahead)
            runner.sched = sch
            reqs = [Req(f"r{i}", p, SamplingParams(max_new_tokens=m, ignore_eos=ignore)) for i, (p, m) in enumerate(zip(prompts, max_new))]
            step, nxt = 0, 0
            while nxt < n or not sch.idle:
                while nxt < n and arrive[nxt] <= step:
                    sch.add_request(reqs[nxt])
                    nxt += 1
                for i, at in abort_at.items():
                    if at == step:
                        sch.abort(f"r{i}")
                sch.step()
                step += 1
                assert step < 5000
            sch.check_idle_invariants()
            assert all(t >= 0 for r in reqs for t in r.tokens)
            results.append([(r.output, r.finish_reason.type) for r in reqs])
        base, look = results
        for i, (b, l) in enumerate(zip(base, look)):
            if i in abort_at:                    # an abort lands a step apart in the two schedules: a prefix either way
                k = min(len(b[0]), len(l[0]))
                assert b[0][:k] == l[0][:k]
            else:
                assert b == l, (trial, i)


def test_scheduler_mixes_decode_tokens_with_prompt_portions():
    prompts = [[3] * 10, [4] * 50]
    reqs, sch, runner = run_all(4, 100, prompts, [30, 5], chunk=16, budget=24, policy="fcfs", prefix_cache=False)
    mixed = [st for st in runner.steps if any(n == 1 for _, n in st) and any(n > 1 for _, n in st)]
    assert mixed, "no step held a decoded token beside a prompt portion"
    assert [n for _, n in runner.steps[0]] == [10, 14]          # budget 24: whole first prompt, portion of the second


def test_prefix_cache_reuse_and_accounting():
    shared = list(range(1, 41))
    prompts = [shared + [50 + i] * 6 for i in range(6)]
    reqs, sch, runner = run_all(4, 200, prompts, [4] * 6, policy="lpm")
    # the first request fills the cache; the others wait for it and then reuse 40 tokens each
    assert reqs[0].cached_tokens == 0
    assert [r.cached_tokens for r in reqs[1:]] == [40] * 5
    assert sch.stats["cached_tokens"] == 200
    assert sch.tree.protected_pages == 0 and sch.tree.num_nodes == sch.mgr.groups[0].pool.in_use
    assert sch.flush_cache() and sch.mgr.groups[0].pool.in_use == 0


def test_pages_run_out_retract_and_finish_everything():
    prompts = prompts_for(3, 6, 20, 30)
    max_new = [40] * 6
    want = [r.output for r in run_all(4, 4000, prompts, max_new, policy="fcfs", prefix_cache=False)[0]]
    # 6 requests want about 6 * 65 tokens; the pool holds 160: optimistic admission must retract
    reqs, sch, runner = run_all(4, 40, prompts, max_new, policy="fcfs", prefix_cache=False, conservativeness=0.3)
    assert sch.stats["retractions"] > 0
    assert [r.output for r in reqs] == want
    assert any(r.retractions for r in reqs)
    assert sch.new_token_ratio > sch.min_ratio


def test_request_that_can_never_fit_is_aborted_not_hung():
    reqs, sch, _ = run_all(4, 8, [[5] * 100, [6] * 10], [4, 4], policy="fcfs", prefix_cache=False)
    assert reqs[0].finish_reason.type == "abort" and "does not fit" in reqs[0].finish_reason.detail
    assert reqs[1].finish_reason.type == "length" and len(reqs[1].output) == 4
    # a lone request that outgrows the pool while decoding is finished with abort as well
    reqs, sch, _ = run_all(4, 8, [[5] * 20], [100], policy="fcfs", prefix_cache=False)
    assert reqs[0].finish_reason.type == "abort" and 0 < len(reqs[0].output) < 100


def test_finish_reasons_and_abort():
    mgr = CacheManager({0: PagedKVNeed(2, 16)}, page_size=4, num_pages=100, max_reqs=4, max_context_len=64)
    runner = FakeRunner(mgr)
    sch = Scheduler(runner, ArgmaxSampler(), policy="fcfs", eos_ids=[9])
    runner.sched = sch
    r_len = Req("a", [1, 2, 3], SamplingParams(max_new_tokens=2))
    r_ctx = Req("b", [1] * 60, SamplingParams(max_new_tokens=50, ignore_eos=True))
    r_abort = Req("c", [4, 5], SamplingParams(max_new_tokens=50))
    r_long = Req("d", [1] * 64, SamplingParams())
    for r in (r_len, r_ctx, r_abort, r_long):
        sch.add_request(r)
    assert r_long.finish_reason.type == "abort"                 # prompt fills the whole context
    sch.step()
    sch.abort("c")
    while not sch.idle:
        sch.step()
    assert r_len.finish_reason.type == "length" and len(r_len.output) == 2
    assert r_ctx.finish_reason.type == "length" and len(r_ctx.output) == 5   # 60 + 5 - 1 = 64 tokens in the cache
    assert r_abort.finish_reason.type == "abort"
    sch.check_idle_invariants()
    # eos: make the fake model emit the eos id
    class Eos(ArgmaxSampler):
        def sample(self, logits, *a):
            return torch.full((logits.shape[0],), 9)
    sch = Scheduler(runner, Eos(), policy="fcfs", eos_ids=[9])
    runner.sched = sch
    r_eos = Req("e", [1, 2], SamplingParams(max_new_tokens=10))
    r_ign = Req("f", [1, 2], SamplingParams(max_new_tokens=3, ignore_eos=True))
    sch.add_request(r_eos)
    sch.add_request(r_ign)
    while not sch.idle:
        sch.step()
    assert r_eos.finish_reason.type == "stop" and r_eos.output == [9]
    assert r_ign.finish_reason.type == "length" and r_ign.output == [9, 9, 9]


def test_policies_order():
    mgr = CacheManager({0: PagedKVNeed(2, 16)}, page_size=4, num_pages=1000, max_reqs=16, max_context_len=512)
    sch = Scheduler(FakeRunner(mgr), ArgmaxSampler(), policy="lof")
    for i, m in enumerate([5, 50, 20]):
        sch.add_request(Req(f"r{i}", [1 + i] * 8, SamplingParams(max_new_tokens=m)))
    assert [r.rid for r, _, _ in sch._ordered_waiting()] == ["r1", "r2", "r0"]
    with pytest.raises(ValueError, match="dfs-weight"):
        Scheduler(FakeRunner(mgr), ArgmaxSampler(), policy="dfs-weight")


# ---------------------------------------------------------------------------------------
# the step function's plan of kv splits (pure arithmetic on the host)
# ---------------------------------------------------------------------------------------
def test_kv_split_plan():
    from mini_sglang_b200.engine.step import MIN_KEYS_PER_PIECE, MIN_KEYS_PER_SPLIT, plan_kv_splits
    SM_COUNT = 148                     # a B200's
    geo = dict(n_kv=8, group=4, blocks_per_sm=4, tile_tokens=2, window=None, sm_count=SM_COUNT)
    slots = SM_COUNT * 4
    # few requests: everybody is cut alike, so that the blocks fill the SMs once
    # (9 blocks a request would fill the 592 places, but 4,096 keys are 256 units of 16 for 4 warps: 8 blocks are as fast)
    ns = plan_kv_splits([1] * 8, [4096] * 8, cap=16, **geo)
    assert slots // 64 == 9 and ns == [8] * 8
    assert plan_kv_splits([1] * 8, [4096 + 16 * 4 * 8] * 8, cap=16, **geo) == [9] * 8
    # a cut never leaves pieces shorter than MIN_KEYS_PER_SPLIT, and a cap holds
    assert plan_kv_splits([1], [3 * MIN_KEYS_PER_SPLIT + 5], cap=16, **geo) == [3]
    assert plan_kv_splits([1] * 8, [4096] * 8, cap=4, **geo) == [4] * 8
    assert plan_kv_splits([1] * 8, [4096] * 8, cap=1, **geo) == [1] * 8
    # as many requests of like length as the GPU holds blocks: nothing is cut
    assert plan_kv_splits([1] * 64, [4096] * 64, cap=1, long_cap=8, **geo) == [1] * 64
    assert plan_kv_splits([1] * 64, [4000 + 3 * i for i in range(64)], cap=1, long_cap=8, **geo) == [1] * 64
    # ... unless the contexts are long and the blocks fall unevenly on the SMs (512 blocks: 3.5 an SM): then halves (1,024: 6.9)
    assert plan_kv_splits([1] * 64, [8192] * 64, cap=1, long_cap=8, **geo) == [2] * 64
    assert plan_kv_splits([1] * 64, [8192] * 64, cap=1, long_cap=1, **geo) == [1] * 64
    assert plan_kv_splits([1] * 72, [8192] * 72, cap=1, long_cap=8, **geo) == [1] * 72        # 576 blocks: 3.9 an SM already
    # fewer blocks than the GPU holds: every request is longer than 1.5 mean loads of a block and is halved (measured better)
    assert plan_kv_splits([1] * 40, [4096] * 40, cap=1, long_cap=8, **geo) == [2] * 40
    # one request far longer than the rest is cut into pieces of about the mean load of a block, the others stay whole
    ns = plan_kv_splits([1] * 65, [1200] + [20] * 64, cap=1, long_cap=8, **geo)
    assert ns[0] == 1200 // MIN_KEYS_PER_PIECE and ns[1:] == [1] * 64
    ns = plan_kv_splits([1] * 48, [8192] + [1024] * 47, cap=1, long_cap=8, **geo)
    assert 2 <= ns[0] <= 8 and ns[1:] == [1] * 47
    # runs longer than one decode tile go whole to the prefill kernels, whatever their length; they do not count as load
    ns = plan_kv_splits([1, 5, 1], [8192, 8192, 200], cap=16, **geo)
    assert ns[1] == 1 and ns[0] > 1 and ns[2] == 1
    # a window bounds the keys that count
    geo_w = dict(geo, window=512)
    # 513 keys: at most 513 // MIN_KEYS_PER_SPLIT = 4 pieces; 33 units of 16 keys are 3 a warp in 3 pieces as in 4
    assert plan_kv_splits([1] * 8, [4096] * 8, cap=16, **geo_w) == [3] * 8
    # wide groups take several blocks per kv head: fewer splits fill the SMs
    wide = dict(n_kv=2, group=32, blocks_per_sm=4, tile_tokens=1, window=None, sm_count=SM_COUNT)
    assert plan_kv_splits([1] * 16, [8192] * 16, cap=16, **wide) == [slots // (16 * 2 * 2)] * 16


def walk_even_cut(cut, n_req):
    """The runs of keys that the blocks of an even cut take, found the way the kernel finds them: per request the list of
    (piece, first unit, end unit) in units of the request."""
    n, start, blk_req, cum, first_blk, pieces = cut
    runs = [[] for _ in range(n_req)]
    for j in range(n):
        lo, hi, r = int(start[j]), int(start[j + 1]), int(blk_req[j])
        while lo < hi:
            c0, c1 = int(cum[r]), int(cum[r + 1])
            assert c0 <= lo < c1
            end = min(hi, c1)
            runs[r].append((j - int(first_blk[r]), lo - c0, end - c0))
            lo, r = end, r + 1
    return runs


def test_even_cut_of_a_decode_step():
    """Every unit of every request lies in exactly one run, the runs of a request are its pieces 0, 1, ... in order, no
    request has more pieces than allowed, and the blocks' loads differ by little."""
    from mini_sglang_b200.engine.step import EVEN_MIN_UNITS, EVEN_SNAP_UNITS, pack_even_cut, plan_even_cut
    n, start, blk_req, cum, first_blk, pieces = plan_even_cut([4096] * 8, None, 74, 32)
    assert n == 74 and cum[-1] == 8 * 256 and pieces.tolist() == [10] * 8
    assert max(np.diff(start)) - min(np.diff(start)) <= 2 * EVEN_SNAP_UNITS + 1
    n, start, *_ , pieces = plan_even_cut([32768], None, 74, 32)              # one request: as many pieces as allowed
    assert n == 32 and pieces.tolist() == [32] and set(np.diff(start).tolist()) == {64}
    n, *_, pieces = plan_even_cut([4096], None, 74, 32)                       # no run below EVEN_MIN_UNITS
    assert n == 256 // EVEN_MIN_UNITS and pieces.tolist() == [n]
    n, *_, pieces = plan_even_cut([5, 1, 30], None, 74, 32)                   # a step smaller than one run
    assert n == 1 and pieces.tolist() == [1, 1, 1]
    # a window bounds the units that count: 16 + 1 keys end in at most two units
    n, start, blk_req, cum, *_ = plan_even_cut([1000, 5000], 17, 74, 32)
    assert cum.tolist() == [0, 2, 4]
    words = pack_even_cut(plan_even_cut([700, 4096, 50], None, 5, 8), 4, 8)   # captured for 4 requests and 8 blocks
    assert words[0] == 5 and len(words) == 1 + 9 + 8 + 5 + 4 and words[1 + 5] == words[1 + 8] == 44 + 256 + 4
    rnd = np.random.RandomState(5)
    for _ in range(300):
        B = int(rnd.randint(1, 130))
        lens = rnd.randint(1, int(rnd.choice([40, 700, 5000, 40000])), B)
        window = None if rnd.rand() < 0.7 else int(rnd.randint(1, 3000))
        blocks, most = int(rnd.choice([1, 3, 18, 37, 74, 148])), int(rnd.choice([1, 2, 8, 32]))
        cut = plan_even_cut(lens, window, blocks, most)
        n, start, blk_req, cum, first_blk, pieces = cut
        assert 1 <= n <= blocks and start[0] == 0 and start[n] == cum[-1] and (np.diff(start) > 0).all()
        assert pieces.max() <= most or n == 1
        for r, runs in enumerate(walk_even_cut(cut, B)):
            assert [p for p, _, _ in runs] == list(range(int(pieces[r])))
            assert runs[0][1] == 0 and runs[-1][2] == cum[r + 1] - cum[r]
            assert all(a[2] == b[1] for a, b in zip(runs, runs[1:]))


def test_which_decode_steps_take_the_even_cut():
    """Requests of like length, short requests and a switched-off cut keep the cut per request; long requests of
    different lengths take the even cut; a window bounds the keys that count."""
    from types import SimpleNamespace
    from mini_sglang_b200.engine.step import ModelRunner
    def wants(lens, window=None):
        stub = SimpleNamespace(mgr=SimpleNamespace(groups=[SimpleNamespace(window=window)]))
        return ModelRunner._wants_even_cut(stub, lens)
    assert not wants([4096] * 8) and not wants([4096 + 3 * i for i in range(64)]) and not wants([32768])
    assert wants([1000 + 1000 * i for i in range(16)]) and wants([30000] + [1000] * 15) and wants([8000] * 4 + [500] * 28)
    assert not wants([64 + 10 * i for i in range(128)])              # 64...1,334 keys: 44 units in the mean
    assert not wants([30000] + [1000] * 15, window=1000)             # every request within its window: alike
    os.environ["MSGL_EVEN_CUT"] = "0"
    try:
        assert not wants([30000] + [1000] * 15)
    finally:
        del os.environ["MSGL_EVEN_CUT"]


def test_order_of_a_decode_batch():
    """The attention launch of a decode step takes the requests by falling number of keys per kv split; rows of equal
    load keep their order, padding rows of a captured batch size come last."""
    from mini_sglang_b200.engine.step import decode_order
    assert decode_order([100, 700, 100, 30], [1, 1, 1, 1], None, 4).tolist() == [1, 0, 2, 3]
    assert decode_order([100, 700, 100, 30], [1, 8, 1, 1], None, 4).tolist() == [0, 2, 1, 3]        # 700 keys in 8 pieces: 88 a block
    assert decode_order([100, 700, 100, 30], [1, 1, 1, 1], 63, 6).tolist() == [0, 1, 2, 3, 4, 5]    # a window of 63: 64, 64, 64, 30 keys
    assert decode_order([5, 9], [1, 1], None, 4).tolist() == [1, 0, 2, 3]
    rnd = np.random.RandomState(3)
    for _ in range(20):
        n, b = int(rnd.randint(1, 40)), 48
        lens, ns = rnd.randint(1, 3000, n), rnd.randint(1, 5, n)
        order = decode_order(lens, ns, None, b).tolist()
        assert sorted(order) == list(range(b)) and order[n:] == list(range(n, b))
        load = [-(-int(lens[i]) // int(ns[i])) for i in order[:n]]
        assert load == sorted(load, reverse=True)


# ---------------------------------------------------------------------------------------
# prefix cache under pressure, portions, and several groups
# ---------------------------------------------------------------------------------------
def make_sched(needs, page_size, num_pages, *, max_reqs=8, budget=16384, chunk=8192, policy="fcfs", **kw):
    mgr = CacheManager(needs, page_size=page_size, num_pages=num_pages, max_reqs=max_reqs, max_context_len=4096,
                       max_step_tokens=budget)
    runner = FakeRunner(mgr)
    sch = Scheduler(runner, ArgmaxSampler(), max_num_reqs=max_reqs, max_step_tokens=budget, chunk_size=chunk,
                    policy=policy, eos_ids=[0], retract_decode_steps=4, **kw)
    runner.sched = sch
    return sch, runner


def drain(sch, limit=20000):
    n = 0
    while not sch.idle:
        sch.step()
        n += 1
        assert n < limit, "scheduler does not make progress"
    sch.check_idle_invariants()


def test_admission_evicting_a_prefix_that_a_later_request_matched():
    """Three requests wait; making room for the first evicts cached pages that the other two matched a
    moment earlier.  Those two must not adopt the evicted pages (the first request owns them now)."""
    X, Z = list(range(1, 13)), list(range(21, 33))
    for policy in ("fcfs", "lpm"):
        sch, runner = make_sched({0: PagedKVNeed(2, 16)}, 4, 42, policy=policy)
        for i, p in enumerate((X, Z)):
            sch.add_request(Req(f"warm{i}", p + [40 + i], SamplingParams(max_new_tokens=2, ignore_eos=True)))
        drain(sch)
        assert sch.tree.num_nodes == 6 and sch.tree.match(X)[0] and sch.tree.match(Z)[0]
        a = Req("a", [50 + i % 9 for i in range(150)], SamplingParams(max_new_tokens=2, ignore_eos=True))
        b = Req("b", X + [45, 46], SamplingParams(max_new_tokens=2, ignore_eos=True))
        c = Req("c", Z + [47, 48], SamplingParams(max_new_tokens=2, ignore_eos=True))
        order = (a, b, c) if policy == "fcfs" else (b, c, a)
        for r in order:
            sch.add_request(r)
        drain(sch)                                           # FakeRunner asserts on every read and on page ownership
        assert sch.stats["evicted_pages"] > 0
        assert all(r.finish_reason.type == "length" and len(r.output) == 2 for r in (a, b, c))


def test_lock_refuses_an_evicted_node():
    tree = PrefixTree(2)
    tree.insert([1, 2, 3, 4], [5, 6], 0)
    _, node = tree.match([1, 2, 3, 4])
    assert tree.evict(2) == [6, 5]
    with pytest.raises(RuntimeError, match="no longer in the tree"):
        tree.lock(node)
    assert tree.evictable_pages == 0 and tree.protected_pages == 0


def test_prompt_portions_reach_the_prefix_cache_one_by_one():
    """Two requests share 64 tokens; prompts are fed 16 tokens a step.  The first one's full pages go to the
    prefix cache after every portion, and the second starts as soon as the shared pages are there: it takes
    all 64 tokens from the cache and never waits for the rest of the first one's prompt."""
    shared = [1 + i % 50 for i in range(64)]
    first = Req("first", shared + [51] * 70, SamplingParams(max_new_tokens=3, ignore_eos=True))
    second = Req("second", shared + [52] * 9, SamplingParams(max_new_tokens=3, ignore_eos=True))
    sch, runner = make_sched({0: PagedKVNeed(2, 16)}, 4, 200, chunk=16, budget=64, policy="lpm")
    sch.add_request(first)
    sch.add_request(second)
    started_at = None
    for step in range(200):
        if sch.idle:
            break
        sch.step()
        if step < 4:
            assert sch.tree.num_nodes == 4 * (step + 1)              # 16 tokens = 4 pages more after every portion
        if started_at is None and second.slot is not None:
            started_at = step
            assert int(sch.mgr.length[first.slot]) < first.n_prompt   # the first prompt is still under way
    assert started_at == 4 and second.cached_tokens == 64
    assert len(first.output) == 3 and len(second.output) == 3
    sch.check_idle_invariants()
    # same tokens as without any sharing
    base = []
    for r in (first, second):
        sch2, _ = make_sched({0: PagedKVNeed(2, 16)}, 4, 200, enable_prefix_cache=False)
        q = Req(r.rid, r.tokens[:r.n_prompt], SamplingParams(max_new_tokens=3, ignore_eos=True))
        sch2.add_request(q)
        drain(sch2)
        base.append(q.output)
    assert [first.output, second.output] == base


def test_scheduler_on_a_model_with_an_all_keys_group_and_a_windowed_group():
    """Admission, retraction and give-backs count every group's pool: here the windowed group's pool is the
    scarce one.  Everything finishes with the tokens of an unconstrained run, no page is lost and nothing starves."""
    needs = {0: PagedKVNeed(2, 16), 1: PagedKVNeed(2, 16, window=12), 2: StateNeed((4,))}
    prompts = prompts_for(5, 10, 10, 70)
    max_new = [5 + (3 * i) % 25 for i in range(10)]

    def run(num_pages, shrink_window_pool=None, **kw):
        sch, runner = make_sched(needs, 4, num_pages, max_reqs=6, budget=40, chunk=16, **kw)
        assert sch.tree is None and len(sch.mgr.groups) == 2
        if shrink_window_pool:
            g = sch.mgr.groups[1]
            g.pool = PagePool(shrink_window_pool)
        reqs = [Req(f"r{i}", p, SamplingParams(max_new_tokens=m, ignore_eos=True)) for i, (p, m) in enumerate(zip(prompts, max_new))]
        for r in reqs:
            sch.add_request(r)
        drain(sch)
        for g in sch.mgr.groups:
            assert g.pool.in_use == 0
        return reqs, sch, runner

    base, sch0, _ = run(4000)
    assert sch0.stats["retractions"] == 0
    # all-keys pool short
    reqs, sch, _ = run(60, conservativeness=0.3)
    assert [r.output for r in reqs] == [r.output for r in base]
    # windowed pool short (14 pages; a request being fed 16 tokens a step holds up to (12 + 16) / 4 + 1 = 8 of them
    # there): admission counts that pool too, so nobody is let in only to be thrown out again
    reqs, sch, runner = run(4000, shrink_window_pool=14)
    assert [r.output for r in reqs] == [r.output for r in base]
    assert sch.stats["retractions"] == 0, "admission ignored the windowed group's pool"
    assert max(len(st) for st in runner.steps) <= 4
    assert all(r.finish_reason.type == "length" for r in reqs)


def test_random_prefix_sharing_under_pressure_gives_the_tokens_of_an_unshared_run():
    """Many random runs: families of prompts that share prefixes of different lengths, prompts fed in small portions, pools so
    small that cached pages are evicted and requests retracted, requests arriving over time, both policies that use the
    prefix cache.  Every run must give each request the tokens it gets alone without any sharing; the stand-in runner checks
    on every step that every page a request reads holds that request's own tokens."""
    rnd = random.Random(5)
    for trial in range(40):
        P = rnd.choice([1, 4, 16])
        n = rnd.randrange(4, 12)
        families = [[rnd.randrange(1, 60) for _ in range(rnd.randrange(8, 70))] for _ in range(rnd.randrange(1, 4))]
        prompts = []
        for i in range(n):
            fam = rnd.choice(families)
            keep = rnd.randrange(0, len(fam) + 1)
            prompts.append(fam[:keep] + [rnd.randrange(1, 60) for _ in range(rnd.randrange(1, 30))])
        max_new = [rnd.randrange(1, 20) for _ in range(n)]
        arrive = sorted(rnd.randrange(0, 25) for _ in range(n))
        longest = max(len(p) + m for p, m in zip(prompts, max_new))
        pages = -(-longest // P) + rnd.randrange(2, 40 // P + 6)
        chunk = rnd.choice([5, 16, 64])
        kw = dict(max_reqs=rnd.choice([2, 4, 8]), budget=rnd.choice([24, 64]), chunk=chunk, policy=rnd.choice(["lpm", "fcfs"]),
                  conservativeness=rnd.choice([0.3, 1.0]), lookahead=rnd.random() < 0.5)
        # every request alone, nothing shared
        want = []
        for p, m in zip(prompts, max_new):
            sch0, _ = make_sched({0: PagedKVNeed(2, 16)}, P, 400, enable_prefix_cache=False)
            q = Req("solo", p, SamplingParams(max_new_tokens=m, ignore_eos=True))
            sch0.add_request(q)
            drain(sch0)
            want.append(q.output)
        sch, runner = make_sched({0: PagedKVNeed(2, 16)}, P, pages, **kw)
        reqs = [Req(f"r{i}", p, SamplingParams(max_new_tokens=m, ignore_eos=True)) for i, (p, m) in enumerate(zip(prompts, max_new))]
        step, nxt = 0, 0
        while nxt < n or not sch.idle:
            while nxt < n and arrive[nxt] <= step:
                sch.add_request(reqs[nxt])
                nxt += 1
            sch.step()
            step += 1
            assert step < 20000, (trial, kw)
        sch.check_idle_invariants()
        assert [r.output for r in reqs] == want, (trial, P, pages, kw)
        assert all(r.finish_reason.type == "length" for r in reqs)


def test_a_lone_decoding_request_is_not_given_up_while_a_prompt_under_way_holds_pages():
    """One request decodes, another is still being fed its prompt in small portions, and the pool runs dry.  The request
    whose prompt is under way (it has produced nothing yet) gives its pages back and waits; nobody is aborted, and everybody
    gets the tokens of an unconstrained run."""
    first = [3 + i % 40 for i in range(10)]
    second = [7 + i % 31 for i in range(30)]
    want = []
    for p, m in ((first, 20), (second, 3)):
        sch0, _ = make_sched({0: PagedKVNeed(2, 16)}, 4, 400, enable_prefix_cache=False)
        q = Req("solo", p, SamplingParams(max_new_tokens=m, ignore_eos=True))
        sch0.add_request(q)
        drain(sch0)
        want.append(q.output)
    # 12 pages = 48 tokens: the first request needs 8 of them at its end, the second 8: admission lets the second in on the
    # estimate that the first will generate a fifth of what it may, and the pool is dry before the second prompt is in
    sch, runner = make_sched({0: PagedKVNeed(2, 16)}, 4, 12, chunk=3, budget=64, conservativeness=0.3, enable_prefix_cache=False)
    a = Req("a", first, SamplingParams(max_new_tokens=20, ignore_eos=True))
    b = Req("b", second, SamplingParams(max_new_tokens=3, ignore_eos=True))
    sch.add_request(a)
    for _ in range(2):
        sch.step()
    sch.add_request(b)
    drain(sch)
    assert sch.stats["aborted"] == 0 and sch.stats["retractions"] >= 1
    assert [a.output, b.output] == want and b.retractions >= 1 and a.retractions == 0


def test_random_runs_on_two_cache_groups_give_the_tokens_of_an_unconstrained_run():
    """Random requests, arrivals, aborts and pool sizes on a model with an all-keys group, a windowed group and per-request
    state: every request that is not aborted gets the tokens of an unconstrained run, and both pools end empty."""
    rnd = random.Random(9)
    needs = {0: PagedKVNeed(2, 16), 1: PagedKVNeed(1, 16, window=10), 2: StateNeed((3,))}
    for trial in range(25):
        P = rnd.choice([1, 4, 8])
        n = rnd.randrange(3, 10)
        prompts = [[rnd.randrange(1, 60) for _ in range(rnd.randrange(1, 60))] for _ in range(n)]
        max_new = [rnd.randrange(1, 25) for _ in range(n)]
        arrive = sorted(rnd.randrange(0, 20) for _ in range(n))
        abort_at = {rnd.randrange(n): rnd.randrange(1, 40)} if trial % 4 == 0 else {}
        longest = max(len(p) + m for p, m in zip(prompts, max_new))
        chunk = rnd.choice([4, 16, 64])
        kw = dict(max_reqs=rnd.choice([2, 4, 6]), budget=rnd.choice([24, 64]), chunk=chunk, conservativeness=rnd.choice([0.3, 1.0]),
                  lookahead=rnd.random() < 0.5)
        want = []
        for p, m in zip(prompts, max_new):
            sch0, _ = make_sched(needs, P, 600, budget=64)
            q = Req("solo", p, SamplingParams(max_new_tokens=m, ignore_eos=True))
            sch0.add_request(q)
            drain(sch0)
            want.append(q.output)
        sch, runner = make_sched(needs, P, -(-longest // P) + rnd.randrange(2, 30), **kw)
        if rnd.random() < 0.5:                       # a scarce windowed pool: room for one request's window and portion, and some
            per_req = -(-(10 + min(chunk, kw["budget"]) + P) // P) + 1
            sch.mgr.groups[1].pool = PagePool(per_req + rnd.randrange(0, 2 * per_req))
        reqs = [Req(f"r{i}", p, SamplingParams(max_new_tokens=m, ignore_eos=True)) for i, (p, m) in enumerate(zip(prompts, max_new))]
        step, nxt = 0, 0
        while nxt < n or not sch.idle:
            while nxt < n and arrive[nxt] <= step:
                sch.add_request(reqs[nxt])
                nxt += 1
            for i, at in abort_at.items():
                if at == step:
                    sch.abort(f"r{i}")
            sch.step()
            step += 1
            assert step < 20000, (trial, kw)
        sch.check_idle_invariants()
        assert all(g.pool.in_use == 0 for g in sch.mgr.groups)
        for i, r in enumerate(reqs):
            if i in abort_at and r.finish_reason.type == "abort":
                assert r.output == want[i][:len(r.output)]
            else:
                assert r.finish_reason.type == "length" and r.output == want[i], (trial, i, P, kw, r.finish_reason)
