"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

Every step is ONE batch for the step function: all running requests that have a single token
to feed (decode) plus portions of prompts, as far as the step's token budget and the free pages
allow.  Roles and rules follow the reference (mini_sglang/managers/scheduler.py:307-448,
mini_sglang/managers/scheduler_policy.py:47-232, mini_sglang/managers/batch_info.py:349-441):

  order       fcfs | lpm (longest cached prefix first; a request that shares its first 32 tokens
              with an earlier waiting or still-prefilling request waits for that one to fill the
              prefix cache) | lof (largest max_new_tokens first) | random
  admission   need = tokens to prefill + (max_new - done) * new_token_ratio must fit into
              free + evictable tokens minus what running and already admitted requests will need
  budget      at most `max_step_tokens` tokens per step; a prompt is fed in portions of at most
              `chunk_size` tokens (the reference prefills whole prompts only)
  pages short evict unpinned prefix-cache pages first; if decoding still does not fit, retract:
              the requests with the fewest generated tokens (ties: longest prompt) give back
              everything they hold and return to the waiting queue with their tokens, until the
              rest can decode `retract_decode_steps` more steps; they are prefilled again later.
              If a single decoding request is left and still does not fit, requests whose prompts
              are still being fed give way first (least in the cache first); if it is alone and still
              does not fit, it is finished with reason abort.
  ratio       new_token_ratio starts at 0.7 * conservativeness, decays to 0.14 of that over 600
              decode steps, and is re-estimated after a retraction.

  overlap     with `lookahead` (and a runner that can take a token from the device) a step's tokens
              are read one call later: while they travel to the host, the next pure-decode step is
              already launched with the sampled tokens taken from device memory, so the GPU never
              waits for the host.  What needs a token's value (a stop token) is seen one step late:
              the request was fed once more, that result is dropped.  Anything else (a waiting
              request, a prompt under way, an abort, pages short) first reads the tokens in flight
              and then plans as usual.  step() then returns the tokens of the step launched by the
              call before.

The scheduler needs of its runner only `mgr` (a CacheManager), `step(entries) -> logits`, and of
its sampler `sample(logits, temperatures, row_keys, steps) -> token ids`; tests drive it with
stand-ins on the CPU.
"""

from __future__ import annotations

import dataclasses
import logging
import random
import time
from typing import Dict, List, Optional, Sequence, Tuple

from ..cache import OutOfPages, PrefixTree
from ..sampling import SamplingParams
from .step import StepEntry

logger = logging.getLogger("mini_sglang_b200.scheduler")
DECODE_LOG_EVERY = 64     # a line for every step with prompt tokens, and for every 64th step without (mini_sglang/managers/scheduler.py:457-491)

IN_BATCH_PREFIX = 32      # tokens two requests must share for the later one to wait (scheduler_policy.py:18-19)


@dataclasses.dataclass
class FinishReason:
    type: str                 # "length" | "stop" | "abort"
    detail: object = None

    def to_json(self):
        if self.type == "length":
            return {"type": "length", "length": self.detail}
        if self.type == "stop":
            return {"type": "stop", "matched": self.detail}
        return {"type": "abort", "message": self.detail}


class Req:
    def __init__(self, rid: str, prompt: Sequence[int], params: SamplingParams, eos_ids: Sequence[int] = ()):
        if len(prompt) == 0:
            raise ValueError("a request needs at least one prompt token")
        self.rid = rid
        self.tokens: List[int] = list(prompt)
        self.n_prompt = len(self.tokens)
        self.params = params
        self.eos_ids = set(eos_ids) if params.eos_token_id == -1 else {params.eos_token_id}
        self.slot: Optional[int] = None
        self.node = None                      # pinned prefix-tree node
        self.cached_tokens = 0                # prompt tokens taken from the prefix cache at first admission
        self.finish_reason: Optional[FinishReason] = None
        self.to_abort: Optional[str] = None
        # what the random draws of this request are keyed by, beside the engine's seed and the step: the request's own
        # seed, or else its number among the requests that its scheduler was given (set there), so that an engine with
        # the same seed and the same requests in the same order draws the same numbers whatever else ran in the process
        self.rng_key: Optional[int] = params.seed
        self.retractions = 0
        self.t_arrive = time.time()
        self.t_first_token: Optional[float] = None

    @property
    def n_output(self) -> int:
        return len(self.tokens) - self.n_prompt

    @property
    def output(self) -> List[int]:
        """The generated tokens that the host has seen (the last entry of `tokens` may stand for a token
        that is still on the device; it is negative then)."""
        out = self.tokens[self.n_prompt:]
        return out[:-1] if out and out[-1] < 0 else out

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None

    def check_finished(self) -> bool:
        """After a token was appended (mini_sglang/managers/req_info.py:123-140)."""
        if self.finish_reason is not None:
            return True
        if self.to_abort is not None:
            self.finish_reason = FinishReason("abort", self.to_abort)
        elif self.n_output >= self.params.max_new_tokens:
            self.finish_reason = FinishReason("length", self.n_output)
        elif not self.params.ignore_eos and self.tokens[-1] in self.eos_ids:
            self.finish_reason = FinishReason("stop", self.tokens[-1])
        return self.finish_reason is not None


class _InFlight:
    """A launched step whose sampled tokens have not been read yet."""

    def __init__(self, reqs, ids, host, event):
        self.reqs: List[Req] = reqs           # the requests sampled in that step, in row order
        self.ids = ids                        # their tokens: device tensor (or anything with tolist())
        self.host = host                      # pinned mirror the copy goes to (None: read `ids` itself)
        self.event = event
        self.placeholder: Dict[str, int] = {}  # rid -> index in req.tokens that stands for this step's token
        self.dead: set = set()                # rids whose token of this step is dropped


@dataclasses.dataclass
class StepOutput:
    req: Req
    token: Optional[int]       # the token sampled for the request in this step (None: aborted before one)
    finished: bool


class Scheduler:
    def __init__(self, runner, sampler, *, max_num_reqs: int = 1024, max_step_tokens: int = 16384,
                 chunk_size: int = 8192, policy: str = "lpm", conservativeness: float = 1.0,
                 retract_decode_steps: int = 20, enable_prefix_cache: bool = True, eos_ids: Sequence[int] = (),
                 init_new_token_ratio: float = 0.7, min_new_token_ratio_factor: float = 0.14,
                 new_token_ratio_decay_steps: int = 600, seed: int = 0, lookahead: bool = False):
        if policy == "dfs-weight":
            raise ValueError("schedule policy dfs-weight is not implemented; choose lpm, fcfs, lof or random")
        if policy not in ("lpm", "fcfs", "lof", "random"):
            raise ValueError(f"unknown schedule policy {policy!r}")
        self.runner, self.sampler = runner, sampler
        self.mgr = runner.mgr
        self.P = self.mgr.page_size
        self.max_num_reqs = min(max_num_reqs, self.mgr.max_reqs)
        self.max_step_tokens = max_step_tokens
        self.chunk_size = max(1, chunk_size)
        self.policy = policy
        self.retract_decode_steps = retract_decode_steps
        self.eos_ids = list(eos_ids)
        can_share = len(self.mgr.groups) == 1 and self.mgr.groups[0].window is None and not self.mgr.state_ids
        self.tree: Optional[PrefixTree] = PrefixTree(self.P) if (enable_prefix_cache and can_share) else None
        if policy == "lpm" and self.tree is None:
            self.policy = "fcfs"
        self.init_ratio = min(init_new_token_ratio * conservativeness, 1.0)
        self.min_ratio = min(self.init_ratio * min_new_token_ratio_factor, 1.0)
        self.ratio_decay = (self.init_ratio - self.min_ratio) / new_token_ratio_decay_steps
        self.new_token_ratio = self.init_ratio
        self.waiting: List[Req] = []
        self.running: List[Req] = []
        self._rand = random.Random(seed)
        self.lookahead = bool(lookahead) and getattr(runner, "supports_device_tokens", False)
        self._inflight: Optional[_InFlight] = None
        self._host_ids = [None, None]         # two pinned buffers for the tokens on their way to the host
        self._host_flip = 0
        self._n_added = 0                      # requests given to add_request so far
        self.stats = {"steps": 0, "decode_tokens": 0, "prefill_tokens": 0, "cached_tokens": 0, "retractions": 0,
                      "evicted_pages": 0, "aborted": 0, "finished": 0}
        self.last_step: Dict[str, object] = {}     # what the last launched step held (for logs and profiles)
        self._decode_steps = 0                     # steps without prompt tokens since the last one with
        self._decode_tokens = 0
        self._decode_t0 = time.time()

    # -- requests --------------------------------------------------------------------------
    def add_request(self, req: Req) -> None:
        self._n_added += 1
        if req.rng_key is None:
            req.rng_key = self._n_added
        limit = self.mgr.max_context_len
        if req.params.eos_token_id == -1 and not req.eos_ids:
            req.eos_ids = set(self.eos_ids)          # the model's own end tokens
        if req.n_prompt >= limit:
            req.finish_reason = FinishReason("abort", f"prompt of {req.n_prompt} tokens does not fit the context of {limit}")
            return
        # the last generated token is never fed, so prompt + max_new - 1 tokens reach the cache
        req.params.max_new_tokens = min(req.params.max_new_tokens, limit - req.n_prompt + 1)
        self.waiting.append(req)

    def abort(self, rid: str, message: str = "aborted") -> None:
        for r in self.waiting + self.running:
            if r.rid == rid:
                r.to_abort = message

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running and self._inflight is None

    # -- accounting ------------------------------------------------------------------------
    def _hold(self, gi: int, n_tokens: float, portion: int = 1) -> float:
        """Tokens' worth of pages of group `gi` that a request of n_tokens holds at most: all of them, or for a
        group that keeps a window the window plus the largest `portion` it is still fed in one step (pages
        behind the window are given back) plus a page for the ragged ends."""
        w = self.mgr.groups[gi].window
        if w is None:
            return n_tokens
        return min(n_tokens, w + portion + self.P)

    def _portion(self, n_unfed: int) -> int:
        return max(1, min(n_unfed, self.chunk_size, self.max_step_tokens))

    def _free_tokens(self, gi: int = 0) -> int:
        ev = self.tree.evictable_pages if (self.tree is not None and gi == 0) else 0
        return (self.mgr.available_pages(gi) + ev) * self.P

    def _claims(self) -> List[float]:
        """Per group: what the running requests will still take (their unfed tokens plus the estimated share of
        the tokens they may still generate)."""
        ratio = self.new_token_ratio
        out = [0.0] * len(self.mgr.groups)
        for r in self.running:
            total = len(r.tokens) + (r.params.max_new_tokens - r.n_output) * ratio
            have = int(self.mgr.length[r.slot])
            portion = self._portion(len(r.tokens) - have)
            for gi in range(len(out)):
                out[gi] += self._hold(gi, total, portion) - self._hold(gi, have, portion)
        return out

    def _make_room(self, pages_per_group: Sequence[int]) -> bool:
        """Evict prefix-cache pages until the pools can hand out `pages_per_group`."""
        for gi, n in enumerate(pages_per_group):
            pool = self.mgr.groups[gi].pool
            if n > pool.available and gi == 0 and self.tree is not None:
                freed = self.tree.evict(n - pool.available)
                if freed:
                    pool.free(freed)
                    self.stats["evicted_pages"] += len(freed)
            if n > pool.available:
                return False
        return True

    def _pages_for(self, plan: Sequence[Tuple[Req, int]]) -> List[int]:
        tot = [0] * len(self.mgr.groups)
        for r, n in plan:
            for gi, k in enumerate(self.mgr.pages_needed(r.slot, n)):
                tot[gi] += k
        return tot

    def _release(self, req: Req, insert: bool) -> None:
        """Give back what a request holds; with `insert`, its full pages go to the prefix cache."""
        if req.slot is None:
            return
        if insert and self.tree is not None:
            self._insert(req)
        self.mgr.close(req.slot)
        if req.node is not None:
            self.tree.unlock(req.node)
            req.node = None
        req.slot = None

    def _insert(self, req: Req) -> None:
        """Offer the request's full pages to the prefix cache; afterwards the request borrows them."""
        slot = req.slot
        n_tok = int(self.mgr.length[slot])
        n_full = n_tok // self.P
        borrowed = int(self.mgr.borrowed[slot])
        if n_full <= borrowed:
            return
        pages = [int(p) for p in self.mgr.block_table_row(0, slot)[:n_full]]
        table, dup, node = self.tree.insert(req.tokens[:n_full * self.P], pages, owned_from=borrowed)
        if dup:
            self.mgr.groups[0].pool.free(dup)
        self.mgr.replace_prefix(slot, table, n_full)
        self.tree.lock(node)
        if req.node is not None:
            self.tree.unlock(req.node)
        req.node = node

    # -- ordering --------------------------------------------------------------------------
    def _ordered_waiting(self) -> List[Tuple[Req, List[int], object]]:
        """Waiting requests in policy order with their prefix match; requests that should wait for
        another one to fill the prefix cache are left out of this step.  The match is a first look for
        the order only: admission matches again, since admitting one request may evict what another matched."""
        matches = {}
        for r in self.waiting:
            if self.tree is not None:
                pages, node = self.tree.match(r.tokens[:-1])
            else:
                pages, node = [], None
            matches[r.rid] = (pages, node)
        order = list(self.waiting)
        if self.policy == "lpm":
            order.sort(key=lambda r: -len(matches[r.rid][0]))          # stable: arrival order among equals
        elif self.policy == "lof":
            order.sort(key=lambda r: -r.params.max_new_tokens)
        elif self.policy == "random":
            self._rand.shuffle(order)
        out = []
        feeding: Dict[tuple, List[Req]] = {}       # requests whose prompt is under way, by their first tokens
        if self.tree is not None:
            for q in self.running:
                if len(q.tokens) >= IN_BATCH_PREFIX and int(self.mgr.length[q.slot]) < len(q.tokens) - 1:
                    feeding.setdefault(tuple(q.tokens[:IN_BATCH_PREFIX]), []).append(q)
        seen = set()
        for r in order:
            pages, node = matches[r.rid]
            if self.tree is not None and len(r.tokens) - 1 >= IN_BATCH_PREFIX:
                key = tuple(r.tokens[:IN_BATCH_PREFIX])
                if self._prefix_on_its_way(r, len(pages) * self.P, feeding.get(key, ())):
                    continue
                if len(pages) * self.P < IN_BATCH_PREFIX:
                    if key in seen:
                        continue                 # an earlier waiting request computes the shared tokens first
                    seen.add(key)
            out.append((r, pages, node))
        return out

    def _prefix_on_its_way(self, r: Req, matched: int, feeding: Sequence[Req]) -> bool:
        """True while a request that is still feeding its prompt has yet to reach whole pages that `r` shares
        with it beyond the `matched` tokens the prefix cache holds now: every portion's full pages go to the
        cache right after its step, so waiting saves `r` from computing them again."""
        P = self.P
        mine = r.tokens[:-1]
        for q in feeding:
            n = min(len(mine), len(q.tokens))
            c = IN_BATCH_PREFIX                 # the caller found the first IN_BATCH_PREFIX tokens equal
            while c < n and mine[c] == q.tokens[c]:
                c += 1
            c = c // P * P
            if c >= IN_BATCH_PREFIX and c > matched and int(self.mgr.length[q.slot]) < c:
                return True
        return False

    # -- retraction ------------------------------------------------------------------------
    def _decode_pages(self, reqs: Sequence[Req], turns: int) -> List[int]:
        tot = [0] * len(self.mgr.groups)
        for r in reqs:
            for gi, k in enumerate(self.mgr.pages_needed(r.slot, turns)):
                tot[gi] += k
        return tot

    def _retract(self, decoding: List[Req]) -> List[Req]:
        """Retract until the rest can decode `retract_decode_steps` more steps
        (mini_sglang/managers/batch_info.py:372-441)."""
        keep = sorted(decoding, key=lambda r: (r.n_output - r.n_prompt), reverse=True)
        retracted = []
        while keep and not self._make_room(self._decode_pages(keep, self.retract_decode_steps)):
            if len(keep) == 1:
                # no other decoding request to take pages from: one more step still has to fit
                if self._make_room(self._decode_pages(keep, 1)):
                    break
                # requests whose prompts are still being fed hold pages too: the one with the least in the cache
                # gives everything back and waits (it has generated nothing yet), before anybody is given up
                feeding = [q for q in self.running if q not in keep and q not in retracted]
                if feeding:
                    q = min(feeding, key=lambda q: int(self.mgr.length[q.slot]))
                    self._release(q, insert=False)
                    q.retractions += 1
                    self.running.remove(q)
                    self.waiting.append(q)
                    retracted.append(q)
                    self.stats["retractions"] += 1
                    continue
                r = keep.pop()
                r.to_abort = "out of cache pages"
                r.check_finished()
                self._release(r, insert=False)
                self.running.remove(r)
                self.stats["aborted"] += 1
                retracted.append(r)
                break
            r = keep.pop()
            self._release(r, insert=False)
            r.retractions += 1
            self.running.remove(r)
            self.waiting.append(r)
            retracted.append(r)
            self.stats["retractions"] += 1
        if keep:
            done = sum(r.n_output for r in keep)
            total = sum(r.params.max_new_tokens for r in keep)
            self.new_token_ratio = min((done + self.retract_decode_steps * len(keep)) / max(total, 1), 1.0)
        return retracted

    # -- one step ----------------------------------------------------------------------------
    def step(self) -> List[StepOutput]:
        outputs: List[StepOutput] = []
        if self._inflight is not None:
            nxt = self._lookahead_rows()
            if nxt:
                return self._step_lookahead(nxt)
            outputs.extend(self._collect(self._inflight, None))
            self._inflight = None
        # aborted before running
        for r in [r for r in self.waiting if r.to_abort is not None]:
            self.waiting.remove(r)
            r.check_finished()
            outputs.append(StepOutput(r, None, True))
            self.stats["aborted"] += 1

        plan: List[Tuple[Req, int]] = []
        budget = self.max_step_tokens

        # 1. decode: every running request with exactly one token to feed
        decoding = [r for r in self.running if len(r.tokens) - int(self.mgr.length[r.slot]) == 1]
        retracted: List[Req] = []
        if decoding:
            if not self._make_room(self._decode_pages(decoding, 1)):
                retracted = self._retract(decoding)
                for r in retracted:
                    if r.finished:
                        outputs.append(StepOutput(r, None, True))
                decoding = [r for r in decoding if r not in retracted]
            else:
                self.new_token_ratio = max(self.new_token_ratio - self.ratio_decay, self.min_ratio)
            decoding = decoding[:budget]
            plan.extend((r, 1) for r in decoding)
            budget -= len(decoding)

        # 2. prompts already under way
        for r in self.running:
            pending = len(r.tokens) - int(self.mgr.length[r.slot])
            if pending <= 1 or budget <= 0 or r in retracted:
                continue
            n = min(pending, self.chunk_size, budget)
            if self._make_room(self._pages_for(plan + [(r, n)])):
                plan.append((r, n))
                budget -= n

        # 3. new requests (none in a step that had to retract)
        if not retracted and budget > 0 and self.waiting:
            ratio = self.new_token_ratio
            n_groups = len(self.mgr.groups)
            used = self._claims()
            for r, _, _ in self._ordered_waiting():
                if len(self.running) >= self.max_num_reqs or budget <= 0 or self.mgr.free_slots == 0:
                    break
                # matched now, not when the order was made: making room for a request admitted earlier in
                # this step may have evicted pages that this one matched then
                pages, node = self.tree.match(r.tokens[:-1]) if self.tree is not None else ([], None)
                prefix = len(pages) * self.P
                extend = len(r.tokens) - prefix
                total = len(r.tokens) + (r.params.max_new_tokens - r.n_output) * ratio
                portion = self._portion(extend)
                need = [self._hold(gi, total, portion) - self._hold(gi, prefix, portion) for gi in range(n_groups)]
                if node is not None:
                    self.tree.lock(node)             # the matched pages are no longer evictable
                free = [self._free_tokens(gi) for gi in range(n_groups)]
                fits = all(need[gi] <= free[gi] - used[gi] for gi in range(n_groups))
                alone = not self.running and not plan
                if not fits and alone and all(self._hold(gi, len(r.tokens) + 1, portion) - self._hold(gi, prefix, portion) <= free[gi]
                                              for gi in range(n_groups)):
                    fits = True          # alone: the estimate of its future length must not keep it out
                if not fits:
                    if node is not None:
                        self.tree.unlock(node)
                    pool_tokens = [g.pool.num_pages * self.P for g in self.mgr.groups]
                    if alone and any(self._hold(gi, len(r.tokens) + 1, portion) > pool_tokens[gi] for gi in range(n_groups)):
                        # alone and still too large for the whole pool: it can never run
                        self.waiting.remove(r)
                        r.to_abort = f"request of {len(r.tokens)} tokens does not fit the cache of {min(pool_tokens)} tokens"
                        r.check_finished()
                        outputs.append(StepOutput(r, None, True))
                        self.stats["aborted"] += 1
                        continue
                    break
                slot = self.mgr.open()
                r.slot, r.node = slot, node
                if pages:
                    self.mgr.adopt_prefix(slot, pages)
                n = min(extend, self.chunk_size, budget)
                if not self._make_room(self._pages_for(plan + [(r, n)])):
                    self._release(r, insert=False)
                    break
                if r.retractions == 0:
                    r.cached_tokens = prefix
                    self.stats["cached_tokens"] += prefix
                self.waiting.remove(r)
                self.running.append(r)
                plan.append((r, n))
                budget -= n
                for gi in range(n_groups):
                    used[gi] += need[gi]

        if not plan and self.running:
            # nobody can move: prompts under way hold the pages and none of them can grow.  The one
            # with the least in the cache gives everything back (or is finished if it is alone).
            victim = min(self.running, key=lambda r: int(self.mgr.length[r.slot]))
            self.running.remove(victim)
            if self.running:
                self._release(victim, insert=False)
                victim.retractions += 1
                self.waiting.append(victim)
                self.stats["retractions"] += 1
            else:
                victim.to_abort = "out of cache pages"
                victim.check_finished()
                self._release(victim, insert=False)
                self.stats["aborted"] += 1
                outputs.append(StepOutput(victim, None, True))
            return outputs
        if not plan:
            return outputs

        # 4. run the batch
        entries, sampled, fed_prompt = [], [], []
        prompt_tokens = cached = 0
        for r, n in plan:
            start = int(self.mgr.length[r.slot])
            last = start + n == len(r.tokens)
            entries.append(StepEntry(r.slot, r.tokens[start:start + n], [n - 1] if last else []))
            if last:
                sampled.append(r)
            if n == 1 and start >= r.n_prompt:
                self.stats["decode_tokens"] += 1
            else:
                self.stats["prefill_tokens"] += n
                prompt_tokens += n
                cached += start
                fed_prompt.append(r)
        logits = self.runner.step(entries)
        self.stats["steps"] += 1
        self._note_step(len(plan), sum(n for _, n in plan), prompt_tokens, cached)
        if self.tree is not None:
            # a prompt's full pages become shareable as soon as the step that computes them is launched
            # (later steps run after it on the same stream), portion by portion
            for r in fed_prompt:
                self._insert(r)
        flight = self._sample(logits, sampled)
        if self.lookahead:
            self._inflight = flight          # read at the next call
        elif flight is not None:
            outputs.extend(self._collect(flight, None))
        for r in [r for r in self.running if r.to_abort is not None and not r.finished]:
            r.check_finished()
            self._release(r, insert=False)
            self.running.remove(r)
            self.stats["aborted"] += 1
            outputs.append(StepOutput(r, None, True))
        return outputs

    # -- what a step held -------------------------------------------------------------------
    def token_usage(self) -> Tuple[int, int, int, float]:
        """(tokens in use, free, evictable, share in use) of the first cache group, in tokens."""
        if not self.mgr.groups:
            return 0, 0, 0, 0.0
        total = self.mgr.groups[0].pool.num_pages * self.P
        free = self.mgr.available_pages(0) * self.P
        ev = (self.tree.evictable_pages if self.tree is not None else 0) * self.P
        used = total - free - ev
        return used, free, ev, used / max(total, 1)

    def _note_step(self, batch: int, n_tokens: int, prompt_tokens: int, cached: int) -> None:
        """Counters of the step just launched, and the log lines: one for every step that feeds prompt
        tokens, one for every DECODE_LOG_EVERY-th step of single tokens."""
        graph = bool(getattr(self.runner, "last_step_used_graph", False))
        self.last_step = {"step": self.stats["steps"], "kind": "extend" if prompt_tokens else "decode", "batch": batch,
                          "tokens": n_tokens, "prompt_tokens": prompt_tokens, "cuda_graph": graph,
                          "waiting": len(self.waiting), "running": len(self.running),
                          "new_token_ratio": round(self.new_token_ratio, 4)}
        if prompt_tokens:
            self._decode_steps = self._decode_tokens = 0
            self._decode_t0 = time.time()
            logger.info("Extend #BS: %d  #Tokens: %d  #PrefixTokens: %d  #ExtendTokens: %d  #DecodeTokens: %d  #waiting-queue: %d",
                        batch, cached + prompt_tokens, cached, prompt_tokens, n_tokens - prompt_tokens, len(self.waiting))
            return
        self._decode_steps += 1
        self._decode_tokens += batch
        if self._decode_steps % DECODE_LOG_EVERY == 1 and logger.isEnabledFor(logging.INFO):
            now = time.time()
            tps = self._decode_tokens / (now - self._decode_t0) if now > self._decode_t0 and self._decode_steps > 1 else 0.0
            used, free, ev, share = self.token_usage()
            self._decode_t0, self._decode_tokens = now, 0
            logger.info("Decode #BS: %d  #Tokens: %d %d %d (%.2f)  #TPS(token/s): %.2f  #CUDA-Graph: %s  #waiting-queue: %d  "
                        "#new-token-ratio: %.3f", batch, used, free, ev, share, tps, graph, len(self.waiting),
                        self.new_token_ratio)

    # -- sampling and results ---------------------------------------------------------------
    def _sample(self, logits, sampled: List[Req]) -> Optional[_InFlight]:
        """Sample one token for every request in `sampled` and start its way to the host."""
        if not sampled:
            return None
        ids = self.sampler.sample(logits, [r.params.temperature for r in sampled],
                                  [r.rng_key for r in sampled], [r.n_output for r in sampled])
        host = event = None
        if self.lookahead and getattr(ids, "is_cuda", False):
            import torch
            k = self._host_flip
            self._host_flip ^= 1
            if self._host_ids[k] is None or self._host_ids[k].numel() < len(sampled):
                self._host_ids[k] = torch.empty(max(1024, len(sampled)), dtype=ids.dtype, pin_memory=True)
            host = self._host_ids[k][:len(sampled)]
            host.copy_(ids, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
        return _InFlight(sampled, ids, host, event)

    def _collect(self, flight: _InFlight, successor: Optional[_InFlight]) -> List[StepOutput]:
        """Read a launched step's tokens and do what follows from them: append, finish, free.
        `successor` is the step launched on top of it (its rows of requests that turn out to be
        finished are dropped)."""
        outputs: List[StepOutput] = []
        if flight.host is not None:
            flight.event.synchronize()
            ids = flight.host.tolist()
        else:
            ids = flight.ids.tolist() if hasattr(flight.ids, "tolist") else list(flight.ids)
        now = time.time()
        for r, tok in zip(flight.reqs, ids):
            if r.rid in flight.dead or r.finished:
                continue
            tok = int(tok)
            at = flight.placeholder.get(r.rid)
            if at is None:
                r.tokens.append(tok)
            else:
                r.tokens[at] = tok
            if r.t_first_token is None:
                r.t_first_token = now
            if r.check_finished():
                if successor is not None:
                    successor.dead.add(r.rid)     # it was fed once more meanwhile: that result is void
                self._release(r, insert=True)
                self.running.remove(r)
                self.stats["finished"] += 1
                outputs.append(StepOutput(r, tok, True))
            else:
                outputs.append(StepOutput(r, tok, False))
        return outputs

    def _lookahead_rows(self) -> List[Tuple[int, Req]]:
        """(row in the step in flight, request) of the requests that the next step can feed before
        that step's tokens are known; empty if the next step needs the usual planning."""
        flight = self._inflight
        if not self.lookahead or flight is None or self.waiting:
            return []
        if any(r.to_abort is not None for r in self.running):
            return []
        live = [(row, r) for row, r in enumerate(flight.reqs) if r.rid not in flight.dead and not r.finished]
        if len(live) != len(self.running) or {id(r) for _, r in live} != {id(r) for r in self.running}:
            return []                             # a prompt is still under way
        # the token in flight is the last one of those that reach max_new_tokens with it
        nxt = [(row, r) for row, r in live if r.n_output + 1 < r.params.max_new_tokens]
        if not nxt or len(nxt) > self.max_step_tokens:
            return []
        if not self._make_room(self._decode_pages([r for _, r in nxt], 1)):
            return []                             # pages short: retraction wants the tokens first
        return nxt

    def _step_lookahead(self, nxt: List[Tuple[int, Req]]) -> List[StepOutput]:
        flight = self._inflight
        self.new_token_ratio = max(self.new_token_ratio - self.ratio_decay, self.min_ratio)
        entries, sampled = [], []
        for row, r in nxt:
            flight.placeholder[r.rid] = len(r.tokens)
            r.tokens.append(-1 - row)             # stands for row `row` of the tokens in flight
            entries.append(StepEntry(r.slot, [-1 - row], [0]))
            sampled.append(r)
        self.stats["decode_tokens"] += len(nxt)
        logits = self.runner.step(entries, prev_ids=flight.ids)
        self.stats["steps"] += 1
        self._note_step(len(nxt), len(nxt), 0, 0)
        successor = self._sample(logits, sampled)
        outputs = self._collect(flight, successor)
        self._inflight = successor
        return outputs

    # -- maintenance -----------------------------------------------------------------------
    def flush_cache(self) -> bool:
        """Forget the prefix cache; only when idle (mini_sglang/managers/scheduler.py:236-255)."""
        if not self.idle:
            return False
        if self.tree is not None:
            pages = self.tree.reset()
            if pages:
                self.mgr.groups[0].pool.free(pages)
        return True

    def check_idle_invariants(self) -> None:
        """No request in flight => every slot is free, every page is free or in the prefix cache, and
        nothing is pinned (mini_sglang/managers/scheduler.py:257-272)."""
        if not self.idle:
            raise RuntimeError("check_idle_invariants called while requests are in flight")
        if self.tree is not None and self.tree.protected_pages:
            raise RuntimeError(f"leak: {self.tree.protected_pages} prefix-cache pages still pinned")
        self.mgr.check_idle(self.tree.num_nodes if self.tree is not None else 0)
