"""The step function: one forward pass over a batch of (request, its next tokens).

    runner.step([StepEntry(slot, tokens, want), ...]) -> float32 logits [wanted, vocab]

Entries are portions of prompts of any length beside single decoded tokens, cut anywhere.  Only
the tokens given are computed; everything earlier is read from the cache that previous steps
left.  The logits come back for the wanted places only, in the order of the entries and of
`want`.  The reference's counterpart is ModelRunner.forward_generate with
BatchInfo.prepare_for_extend / prepare_for_decode (mini_sglang/managers/model_runner.py:193-229,
mini_sglang/managers/batch_info.py:135-302), which runs either prompts or decoded tokens, never
both, and returns the last position only.

Per step the host writes ONE pinned int32 staging buffer (token ids, positions, request
offsets and lengths, request slots, wanted rows, and per cache group the token slots, kv
splits and block-table rows) and copies it to the device with one transfer.  Steps in which
every request brings exactly one token replay a CUDA graph captured for that batch size.
"""

from __future__ import annotations

import dataclasses
import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..cache import CacheManager, OutOfPages, PagedKVNeed, StateNeed
from ..config import ModelSpec, load_config
from ..parts import BuildEnv, DecoderModel, GroupContext, KVCacheView, StateCacheView, StepContext, Workspace
from ..weights import CheckpointSource, RandomSource

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
MAX_KV_SPLIT = 32                 # more than MANY_SPLITS pieces only where they stay long (below)
MANY_SPLITS, MANY_SPLITS_MIN_KEYS = 16, 512      # one request of 32k keys: 16 pieces 4.54, 32 pieces 4.29 ms a step; of 4k keys: 3.37 / 3.44
MIN_KEYS_PER_SPLIT = 128          # 64 / 128 / 256 / 512 measured at 1 to 8 requests of 1k to 4k keys: 128 best or level (batch 1, 4,096 keys: 3.46 against 3.54 ms with 256)
MIN_KEYS_PER_PIECE = 256          # shortest piece when a single long request is cut up among many short ones
EVEN_MIN_UNITS = 16               # an even cut gives no block fewer than this many units of 16 keys (256 keys, as the pieces above)
EVEN_SNAP_UNITS = 4               # a cut this close to a request's edge moves onto it: a run of a few units costs more than it evens out
EVEN_FROM_UNITS = 64              # a decode step takes the even cut from this many units (1,024 keys) a request on in the mean ...
EVEN_UNEVEN = 1.25                # ... if its longest request has this many times the mean or more
EVEN_MAX_PIECES = 48              # most runs that one request lies in (one request of 30,000 keys among 15 of 1,000, 4 layers: 32: 0.846, 48: 0.816, 74: 0.821 ms a step)
LONG_REQUEST_FACTOR = 1.5         # a request beyond this many times the mean load per block is cut up (1.0, 1.25, 1.5 measured: 1.5 best)
BALANCE_MIN_KEYS = 6144           # mean keys a request from which halving every request to even out the SMs pays
WIDE_KV_SPLIT = 8                 # cap of the decode graphs that are captured for batches with such requests


@dataclasses.dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among `tokens` whose logits are wanted


def _align4(n: int) -> int:
    return (n + 3) & ~3


class _Layout:
    """Offsets of the fields inside the int32 staging buffer of a step."""

    def __init__(self, T: int, B: int, W: int, max_pages: Sequence[int], even_nb: Optional[Sequence[int]] = None):
        self.T, self.B, self.W, self.max_pages = T, B, W, list(max_pages)
        self.even_nb = list(even_nb) if even_nb is not None else [0] * len(self.max_pages)      # 0: no even cut for the group
        off = 0

        def take(n):
            nonlocal off
            o = off
            off += _align4(max(n, 1))
            return o

        self.input_ids, self.positions, self.token_req = take(T), take(T), take(T)
        self.q_start, self.kv_len, self.slots, self.want = take(B + 1), take(B), take(B), take(W)
        self.out_loc, self.nsplit, self.order, self.even, self.table = [], [], [], [], []
        for mp, nb in zip(max_pages, self.even_nb):
            self.out_loc.append(take(T))
            self.nsplit.append(take(B))
            self.order.append(take(B))
            self.even.append(take(ops.even_cut_size(B, nb) if nb else 0))
            self.table.append(take(B * mp))
        self.size = off


class CacheStorage:
    """Device arrays behind the cache manager: per cache id K and V [pages + 1, kv heads, page,
    head size] in the activation dtype, or a state array [max requests + 1, ...]."""

    def __init__(self, mgr: CacheManager, dtype: torch.dtype, device):
        self.kv: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.state: Dict[int, torch.Tensor] = {}
        for cid, need in mgr.needs.items():
            if isinstance(need, PagedKVNeed):
                g = mgr.groups[mgr.group_of_cache[cid]]
                shape = (g.pool.num_pages + 1, need.n_kv_heads, mgr.page_size, need.head_dim)
                self.kv[cid] = (torch.zeros(shape, dtype=dtype, device=device), torch.zeros(shape, dtype=dtype, device=device))
            elif isinstance(need, StateNeed):
                dt = {"float32": torch.float32, "compute": dtype, "int32": torch.int32}[need.dtype]
                self.state[cid] = torch.zeros((mgr.max_reqs + 1, *need.shape), dtype=dt, device=device)
        if self.state:
            mgr.on_open.append(self._zero_slot)
        # device copies of the groups' block tables, brought up to date by deltas before a decode graph is replayed
        self.tables = [torch.zeros((mgr.max_reqs + 1, g.table.shape[1]), dtype=torch.int32, device=device) for g in mgr.groups]

    def _zero_slot(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()

    def bytes(self) -> int:
        n = sum(k.numel() * k.element_size() * 2 for k, _ in self.kv.values())
        return n + sum(t.numel() * t.element_size() for t in self.state.values())


def kv_bytes_per_page(needs: Dict[int, object], page_size: int, dtype: torch.dtype) -> int:
    item = torch.empty((), dtype=dtype).element_size()
    return sum(2 * page_size * n.n_kv_heads * n.head_dim * item for n in needs.values() if isinstance(n, PagedKVNeed))


class _Graph:
    def __init__(self):
        self.graph = None
        self.dev = None        # static device staging buffer
        self.layout = None
        self.logits = None
        self.max_split = None
        self.n_kernels = 0     # this engine's kernels inside the captured graph


DECODE_UNIT_KEYS, DECODE_WARPS = 16, 4        # the decode kernel's warps take units of 16 keys in turn


def _fewest_splits_as_fast(keys: int, ns: int, warps: int = DECODE_WARPS) -> int:
    """The smallest number of splits whose busiest warp has no more units of keys than with `ns` splits (fewer
    blocks then leave fewer partial results to merge: 4,096 keys cut for 9 blocks are as fast in 8)."""
    units = -(-keys // DECODE_UNIT_KEYS)

    def per_warp(n: int) -> int:
        return -(-(-(-units // n)) // warps)

    if ns <= 1:
        return max(ns, 1)
    target = per_warp(ns)
    while ns > 1 and per_warp(ns - 1) == target:
        ns -= 1
    return ns


def plan_kv_splits(q_lens: Sequence[int], kv_lens: Sequence[int], *, n_kv: int, group: int, blocks_per_sm: int,
                   tile_tokens: int, window: Optional[int], cap: int, long_cap: Optional[int] = None,
                   sm_count: int, warps: int = DECODE_WARPS) -> List[int]:
    """kv splits per request of one attention launch.  Only query runs that fit one tile of the decode kernel
    (`tile_tokens`) are split (the prefill kernels take whole key ranges).  Two reasons to split: the launch
    would otherwise leave most of the SMs idle (few requests: every request is cut alike), or one request is
    much longer than the launch's mean load per resident block, so that its single block would still run when
    all others are done (it is cut into pieces of about that load).  `cap` bounds the first kind of cut,
    `long_cap` (default: the same) the second.  `sm_count`: the device's number of SMs; `warps`: warps
    of a block of the kernel that will run the launch."""
    long_cap = cap if long_cap is None else long_cap
    if cap <= 1 and long_cap <= 1:
        return [1] * len(q_lens)
    chunks = 1 if group <= 16 else -(-group // 16)
    heads = n_kv * chunks
    slots = sm_count * blocks_per_sm
    blocks = sum(-(-q // tile_tokens) for q in q_lens) * heads
    want = slots // max(blocks, 1)                    # fill the SMs once, not more
    keys = [min(kv, window + q) if window else kv for q, kv in zip(q_lens, kv_lens)]
    load = sum(k for q, k in zip(q_lens, keys) if q <= tile_tokens) * heads / slots      # keys per resident block, dealt out evenly
    piece = max(MIN_KEYS_PER_PIECE, int(load * LONG_REQUEST_FACTOR))
    out = []
    for q, k in zip(q_lens, keys):
        if q > tile_tokens:
            out.append(1)                             # one decode tile at most
            continue
        most = max(min(k // MIN_KEYS_PER_SPLIT, MANY_SPLITS), k // MANY_SPLITS_MIN_KEYS)
        even = _fewest_splits_as_fast(k, min(want, most, cap), warps)
        long_one = min(-(-k // piece), k // MIN_KEYS_PER_PIECE, long_cap) if k > piece else 1      # no piece below the minimum
        out.append(max(1, even, long_one))
    # Many requests of like, long contexts and nothing cut so far: the kernel's time follows the largest number of
    # blocks that one SM gets, so a launch of 3.5 blocks per SM runs as long as one of 4.  Twice as many blocks of half
    # the size even that out; the merge of the halves costs a fixed few microseconds, which pays from about 6,000 keys a
    # request on (64 requests x 8 kv heads, per decode step of 36 layers: 4,096 keys 10.9 -> 11.0 ms, 8,192 keys 18.6 -> 17.7 ms).
    cut = [i for i, q in enumerate(q_lens) if q <= tile_tokens]
    if cut and long_cap >= 2 and all(n == 1 for n in out):
        n_blocks = len(cut) * heads
        uneven = -(-n_blocks // sm_count) * sm_count / n_blocks - 1.0
        uneven_halved = -(-2 * n_blocks // sm_count) * sm_count / (2 * n_blocks) - 1.0
        if uneven >= 0.08 and uneven_halved <= uneven - 0.04 and sum(keys[i] for i in cut) >= BALANCE_MIN_KEYS * len(cut):
            for i in cut:
                if keys[i] >= 2 * MIN_KEYS_PER_PIECE:
                    out[i] = 2
    return out


def plan_even_cut(kv_lens: Sequence[int], window: Optional[int], n_blocks: int, max_pieces: int):
    """The keys of a decode step (one new token a request) dealt out evenly over the blocks of one kv head.

    The requests' units of DECODE_UNIT_KEYS keys (from the first unit a window still reaches to the unit of the newest
    key) are laid end to end and cut into at most `n_blocks` runs of equal length; a cut that falls within
    EVEN_SNAP_UNITS of a request's edge moves onto it.  No run is shorter than EVEN_MIN_UNITS unless the whole step is,
    and no request lies in more than `max_pieces` runs (fewer blocks are used if it would).

    -> (blocks in use n, start unit of every block [n + 1], first request of every block [n], first unit of every
    request [B + 1], first block of every request [B], pieces of every request [B]); int32 arrays."""
    pos = np.asarray(kv_lens, dtype=np.int64) - 1
    k_lo = np.maximum(pos - window + 1, 0) if window else np.zeros_like(pos)
    units = pos // DECODE_UNIT_KEYS - k_lo // DECODE_UNIT_KEYS + 1
    B = len(units)
    cum = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(units, out=cum[1:])
    U = int(cum[-1])
    n = max(1, min(n_blocks, U // EVEN_MIN_UNITS))
    while True:
        raw = (np.arange(n + 1, dtype=np.int64) * U) // n
        snap = min(EVEN_SNAP_UNITS, (U // n) // 4)
        idx = np.clip(np.searchsorted(cum, raw, side="right") - 1, 0, B - 1)          # the request a cut falls into
        below, above = raw - cum[idx], cum[idx + 1] - raw
        start = np.where(below <= snap, cum[idx], np.where(above <= snap, cum[idx + 1], raw))
        start[0], start[n] = 0, U
        first_blk = np.searchsorted(start, cum[:-1], side="right") - 1                  # the run that holds a request's first unit
        last_blk = np.searchsorted(start, cum[1:], side="left") - 1                     # ... and its last
        pieces = last_blk - first_blk + 1
        most = int(pieces.max())
        if most <= max_pieces or n == 1:
            break
        n = max(1, min(n - 1, n * max_pieces // most))
    blk_req = np.searchsorted(cum, start[:-1], side="right") - 1
    i32 = lambda a: np.asarray(a, dtype=np.int32)
    return n, i32(start), i32(blk_req), i32(cum), i32(first_blk), i32(pieces)


def pack_even_cut(cut, B: int, n_blocks: int) -> np.ndarray:
    """The result of plan_even_cut as the words the attention launch reads (ops.even_cut_size(B, n_blocks) of them): B
    and n_blocks are the sizes the launch was captured with, at least the cut's own."""
    n, start, blk_req, cum, first_blk, _ = cut
    out = np.zeros(ops.even_cut_size(B, n_blocks), dtype=np.int32)
    out[0] = n
    o = 1
    out[o:o + n + 1] = start
    out[o + n + 1:o + n_blocks + 1] = start[n]
    o += n_blocks + 1
    out[o:o + n] = blk_req
    o += n_blocks
    out[o:o + len(cum)] = cum
    out[o + len(cum):o + B + 1] = cum[-1]
    o += B + 1
    out[o:o + len(first_blk)] = first_blk
    return out


def decode_order(kv_lens, nsplits, window: Optional[int], b: int) -> np.ndarray:
    """The rows of a decode batch in the order in which the attention launch takes them: by falling number of keys
    per kv split (blocks go to the SMs in index order, so the longest start first and the shortest fill the end);
    ties keep the rows' order, and the padding rows up to `b` come last."""
    keys = np.asarray(kv_lens, dtype=np.int64)
    if window:
        keys = np.minimum(keys, window + 1)
    ns = np.maximum(np.asarray(nsplits, dtype=np.int64), 1)
    load = np.zeros(b, dtype=np.int64)
    load[:len(keys)] = -(-keys // ns)
    return np.argsort(-load, kind="stable").astype(np.int32)


class ModelRunner:
    def __init__(self, spec: ModelSpec, source_factory, *, dtype: str = "bfloat16", page_size: int = 16,
                 num_pages: Optional[int] = None, max_reqs: int = 64, max_context_len: Optional[int] = None,
                 max_step_tokens: int = 8192, gpu_memory_utilization: float = 0.9, device: str = "cuda:0",
                 use_cuda_graph: bool = True, max_capture_bs: int = 128):
        self.device = self._init_device(device)
        self.sm_count = self._sm_count()
        self.dtype = DTYPES[dtype]
        if self.dtype == torch.float32:
            ops.set_true_fp32()
        self.spec = spec
        self.page_size = page_size
        self.max_context_len = min(max_context_len or spec.max_context_len, spec.max_context_len)
        self.max_step_tokens = max_step_tokens
        env = BuildEnv(dtype=self.dtype, device=self.device)
        self.model = DecoderModel(spec, env)
        head_dims = sorted({n.head_dim for n in self.model.cache_needs().values() if isinstance(n, PagedKVNeed)})
        ops.warm_up(head_dims)
        expected = self.model.tensors()
        src = source_factory(expected, self.dtype, self.device)
        try:
            with torch.no_grad():
                self.model.load(src)
        finally:
            src.close()
        needs = self.model.cache_needs()
        if num_pages is None:
            torch.cuda.empty_cache()
            free, total = torch.cuda.mem_get_info(self.device)
            budget = int(total * gpu_memory_utilization) - (total - free)
            per_page = max(kv_bytes_per_page(needs, page_size, self.dtype), 1)
            num_pages = max(budget // per_page, 0)
            num_pages = min(num_pages, max_reqs * (-(-self.max_context_len // page_size)))
            if num_pages < 1:
                raise RuntimeError("no memory left for the cache; lower gpu_memory_utilization's complement or the model size")
        self.mgr = CacheManager(needs, page_size=page_size, num_pages=num_pages, max_reqs=max_reqs,
                                max_context_len=self.max_context_len, max_step_tokens=max_step_tokens)
        self.storage = CacheStorage(self.mgr, self.dtype, self.device)
        self.workspace = Workspace(self.device)
        self.vocab_size = spec.vocab_size
        self._pinned = [None, None]
        self._pinned_ev = [None, None]
        self._flip = 0
        self._dev_staging = None
        self._steps_run = 0
        if self.device.type == "cuda":
            ops._status_tensor(self.device)          # allocated now, not inside a stream capture
        self.use_cuda_graph = use_cuda_graph and all(getattr(l.mixer, "graph_safe", False) and getattr(l.ffn, "graph_safe", True)
                                                     for l in self.model.layers)
        self.max_capture_bs = max_capture_bs
        self._graphs: Dict[Tuple[int, Tuple[int, ...], bool], _Graph] = {}
        self._graph_pool = None
        self.kernel_launches = 0
        self.last_step_used_graph = False
        # decode steps through a graph: the step's fields are made on the device from three numbers a request and the
        # device copy of the block tables (MSGL_DEVICE_META=0: the host writes them all and copies them)
        self.device_meta = os.environ.get("MSGL_DEVICE_META", "1") != "0"
        self._dev_compact = None
        self.last_h2d_bytes = 0          # bytes of the last step's host-to-device copy of its fields
        self.last_plan: Dict[str, object] = {}       # the last step's kv splits per group and the decode graph it replayed
        self._group_geom = []
        for g in self.mgr.groups:
            cid = g.cache_ids[0]
            need = needs[cid]
            G = max(need.q_heads // need.n_kv_heads, 1) if need.q_heads else 1
            qt = ops.attention_tile_tokens(ops.VARIANT_MMA_DECODE, G, need.head_dim) if ops.mma_supported(need.head_dim, self.dtype) \
                else ops.attention_tile_tokens(ops.VARIANT_SIMT, G)
            self._group_geom.append((need.n_kv_heads, G, ops.decode_blocks_per_sm(need.head_dim, self.dtype, G), qt))
        # blocks per kv head of a decode launch with an even cut of the keys: what the SMs hold at once; empty unless the
        # decode kernel of every group takes such a cut
        self._even_nb: List[int] = []
        if self.dtype == torch.bfloat16 and self.mgr.groups:
            ok = True
            for g, (n_kv, G, per_sm, _) in zip(self.mgr.groups, self._group_geom):
                head_dim = needs[g.cache_ids[0]].head_dim
                ok = ok and ops.decode_even_ok(head_dim, self.dtype, G) and self.sm_count * per_sm >= n_kv
            if ok:
                self._even_nb = [max(1, self.sm_count * per_sm // n_kv) for (n_kv, G, per_sm, _) in self._group_geom]

    # -- device ------------------------------------------------------------------------------
    def _init_device(self, device: str) -> torch.device:
        if not torch.cuda.is_available():
            raise RuntimeError("mini_sglang_b200 runs on a CUDA device (B200, sm_100a) only; none is visible")
        dev = torch.device(device)
        torch.cuda.set_device(dev)
        return dev

    def _sm_count(self) -> int:
        return ops.sm_count(self.device)

    def _alloc_pinned(self, n: int) -> torch.Tensor:
        return torch.empty(n, dtype=torch.int32, pin_memory=True)

    def _new_event(self):
        return torch.cuda.Event()

    # -- construction helpers ------------------------------------------------------------
    @classmethod
    def from_model_dir(cls, model_dir: str, **kw) -> "ModelRunner":
        _, spec = load_config(model_dir)
        return cls(spec, lambda exp, dt, dev: CheckpointSource(model_dir, exp, dt, dev), **kw)

    @classmethod
    def from_random(cls, spec: ModelSpec, seed: int, **kw) -> "ModelRunner":
        return cls(spec, lambda exp, dt, dev: RandomSource(exp, seed, dt, dev), **kw)

    # -- request slots -------------------------------------------------------------------
    def open(self) -> int:
        return self.mgr.open()

    def close(self, slot: int) -> None:
        self.mgr.close(slot)

    # -- staging ---------------------------------------------------------------------------
    def _pinned_buffer(self, n: int) -> torch.Tensor:
        i = self._flip
        self._flip ^= 1
        if self._pinned_ev[i] is not None:
            self._pinned_ev[i].synchronize()
        buf = self._pinned[i]
        if buf is None or buf.numel() < n:
            buf = self._alloc_pinned(max(n, 4096))
            self._pinned[i] = buf
        return buf, i

    FUSED_WARPS = 16         # warps of a block of the whole-step decode kernel

    def _fused_blocks(self, tokens: int) -> int:
        """Blocks of the whole-step decode kernel for a step of `tokens` single tokens with all logits wanted; 0 if the
        model or the size goes kernel by kernel."""
        fd = self.model.fused_decode
        if fd is None or not 0 < tokens <= ops.FUSED_DECODE_MAX_TOKENS or len(self.mgr.groups) != 1:
            return 0
        return fd.blocks_for(tokens)

    def _plan_splits(self, gi: int, q_lens: Sequence[int], kv_lens: Sequence[int], cap: int,
                     long_cap: Optional[int] = None, fused_blocks: int = 0) -> List[int]:
        n_kv, G, per_sm, qt = self._group_geom[gi]
        warps = DECODE_WARPS
        if fused_blocks:          # the whole-step kernel: its blocks are the places, a unit is a (request, kv head, split)
            per_sm, warps, qt = max(fused_blocks // self.sm_count, 1), self.FUSED_WARPS, 1
        return plan_kv_splits(q_lens, kv_lens, n_kv=n_kv, group=G, blocks_per_sm=per_sm, tile_tokens=qt,
                              window=self.mgr.groups[gi].window, cap=cap, long_cap=long_cap, sm_count=self.sm_count,
                              warps=warps)

    def _fill(self, host: np.ndarray, lay: _Layout, entries: Sequence[StepEntry], starts: Sequence[int],
              want_rows: Sequence[int], nsplits: Sequence[Sequence[int]], pad_to: int = 0, even_cuts=None) -> None:
        """Write every field of the staging buffer.  Rows beyond len(entries) (graph padding) are
        single tokens of a request of length 1 on the dump page."""
        T, B = lay.T, lay.B
        host[:lay.size] = 0
        n_ent = len(entries)
        for gi in range(len(self.mgr.groups)):
            host[lay.order[gi]: lay.order[gi] + B] = np.arange(B, dtype=np.int32)
        if n_ent and all(len(e.tokens) == 1 for e in entries):
            # one token per request (decode): every field with a handful of vector operations
            slots = np.fromiter((e.slot for e in entries), dtype=np.int64, count=n_ent)
            pos = np.asarray(starts, dtype=np.int64)
            host[lay.input_ids: lay.input_ids + n_ent] = [e.tokens[0] for e in entries]
            host[lay.positions: lay.positions + n_ent] = pos
            host[lay.token_req: lay.token_req + n_ent] = np.arange(n_ent, dtype=np.int32)
            host[lay.q_start: lay.q_start + n_ent] = np.arange(n_ent, dtype=np.int32)
            host[lay.kv_len: lay.kv_len + n_ent] = pos + 1
            host[lay.slots: lay.slots + n_ent] = slots
            P = self.page_size
            for gi, g in enumerate(self.mgr.groups):
                mp = lay.max_pages[gi]
                host[lay.out_loc[gi]: lay.out_loc[gi] + n_ent] = g.table[slots, pos // P].astype(np.int64) * P + pos % P
                host[lay.nsplit[gi]: lay.nsplit[gi] + n_ent] = nsplits[gi]
                host[lay.order[gi]: lay.order[gi] + B] = decode_order(pos + 1, nsplits[gi], g.window, B)
                if lay.even_nb[gi] and even_cuts is not None:
                    words = pack_even_cut(even_cuts[gi], B, lay.even_nb[gi])
                    host[lay.even[gi]: lay.even[gi] + len(words)] = words
                width = min(mp, g.table.shape[1])
                host[lay.table[gi]: lay.table[gi] + n_ent * mp].reshape(n_ent, mp)[:, :width] = g.table[slots, :width]
            t = n_ent
        else:
            t = 0
            for r, (e, s) in enumerate(zip(entries, starts)):
                n = len(e.tokens)
                host[lay.input_ids + t: lay.input_ids + t + n] = e.tokens
                host[lay.positions + t: lay.positions + t + n] = np.arange(s, s + n, dtype=np.int32)
                host[lay.token_req + t: lay.token_req + t + n] = r
                host[lay.q_start + r] = t
                host[lay.kv_len + r] = s + n
                host[lay.slots + r] = e.slot
                for gi in range(len(self.mgr.groups)):
                    host[lay.out_loc[gi] + t: lay.out_loc[gi] + t + n] = self.mgr.slot_mapping(gi, e.slot, s, n)
                    row = self.mgr.block_table_row(gi, e.slot)
                    mp = lay.max_pages[gi]
                    host[lay.table[gi] + r * mp: lay.table[gi] + r * mp + len(row)] = row
                    host[lay.nsplit[gi] + r] = nsplits[gi][r]
                t += n
        for r in range(len(entries), B):          # padding rows of a captured batch size
            host[lay.token_req + t] = r
            host[lay.q_start + r] = t
            host[lay.kv_len + r] = 1
            for gi in range(len(self.mgr.groups)):
                host[lay.nsplit[gi] + r] = 1
            t += 1
        host[lay.q_start + B] = t
        host[lay.want: lay.want + len(want_rows)] = want_rows

    def _context(self, dev: torch.Tensor, lay: _Layout, q_lens, kv_lens, slots, max_splits, uniform: bool,
                 nsplits=None, all_rows_wanted: bool = False) -> StepContext:
        def v(off, n):
            return dev[off: off + n]

        groups = []
        for gi, g in enumerate(self.mgr.groups):
            mp = lay.max_pages[gi]
            groups.append(GroupContext(block_table=v(lay.table[gi], lay.B * mp).view(lay.B, mp),
                                       out_loc=v(lay.out_loc[gi], lay.T),
                                       nsplit=v(lay.nsplit[gi], lay.B) if max_splits[gi] > 1 else None,
                                       max_split=max_splits[gi], window=g.window,
                                       host_nsplit=nsplits[gi] if nsplits is not None else None,
                                       order=v(lay.order[gi], lay.B) if uniform else None,
                                       even=v(lay.even[gi], ops.even_cut_size(lay.B, lay.even_nb[gi])) if uniform and lay.even_nb[gi] else None,
                                       even_nb=lay.even_nb[gi] if uniform else 0))
        return StepContext(T=lay.T, B=lay.B, page_size=self.page_size, input_ids=v(lay.input_ids, lay.T),
                           positions=v(lay.positions, lay.T), q_start=v(lay.q_start, lay.B + 1),
                           kv_len=v(lay.kv_len, lay.B), token_req=v(lay.token_req, lay.T), slots=v(lay.slots, lay.B),
                           groups=groups, host_q_lens=list(q_lens), host_kv_lens=list(kv_lens),
                           host_slots=list(slots), uniform_decode=uniform, all_rows_wanted=all_rows_wanted,
                           workspace=self.workspace)

    def _caches(self, ctx: StepContext) -> Dict[int, object]:
        views: Dict[int, object] = {}
        for cid, (k, v) in self.storage.kv.items():
            views[cid] = KVCacheView(k, v, ctx.groups[self.mgr.group_of_cache[cid]], self.page_size)
        for cid, st in self.storage.state.items():
            views[cid] = StateCacheView(st)
        return views

    # -- the step ----------------------------------------------------------------------------
    def pages_short(self, entries: Sequence[StepEntry]) -> List[int]:
        """Per group: how many pages the step needs beyond what is free (all zeros: it fits)."""
        need = [0] * len(self.mgr.groups)
        for e in entries:
            for gi, n in enumerate(self.mgr.pages_needed(e.slot, len(e.tokens))):
                need[gi] += n
        return [max(0, n - g.pool.available) for n, g in zip(need, self.mgr.groups)]

    supports_device_tokens = True

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry], prev_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run one batch.  With `prev_ids` (int32 on the device, e.g. the tokens a sampler just wrote), a
        token id -1 - r in an entry stands for prev_ids[r]: it is put in place on the device, so the host
        need not have seen it."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        V = self.vocab_size
        lowest = -int(prev_ids.numel()) if prev_ids is not None else 0        # -1 - r: row r of prev_ids, on the device
        if all(len(e.tokens) == 1 for e in entries):          # a decode batch: one look at all tokens
            toks = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=len(entries))
            if toks.min() < lowest or toks.max() >= V:
                bad = next(e for e in entries if not lowest <= e.tokens[0] < V)
                raise ValueError(f"token id outside [0, {V}) in the entry of slot {bad.slot}")
        else:
            for e in entries:
                toks = np.asarray(e.tokens)
                if toks.min() < lowest or toks.max() >= V:
                    raise ValueError(f"token id outside [0, {V}) in the entry of slot {e.slot}")
        for e in entries:
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"wanted place {w} is outside the entry's {len(e.tokens)} tokens")
        short = self.pages_short(entries)
        if any(short):
            raise OutOfPages(f"the step needs {short} more pages than are free (per group)")
        starts = [int(self.mgr.length[e.slot]) for e in entries]
        for e in entries:
            self.mgr.reserve(e.slot, len(e.tokens))
        q_lens = [len(e.tokens) for e in entries]
        kv_lens = [s + n for s, n in zip(starts, q_lens)]
        want_rows, t = [], 0
        for e in entries:
            want_rows.extend(t + w for w in e.want)
            t += len(e.tokens)
        T, B = t, len(entries)
        uniform = all(n == 1 for n in q_lens)
        all_last = uniform and len(want_rows) == B and all(len(e.want) == 1 for e in entries)

        # kernels with bounded waits report through a status word: look at the last copy of it that has
        # arrived, and queue a fresh one after this step (every step with prompt portions, else now and then)
        ops.raise_if_failed()
        self._steps_run += 1
        self.last_step_used_graph = bool(self.use_cuda_graph and all_last and B <= self.max_capture_bs)
        if self.last_step_used_graph:
            logits = self._step_graph(entries, starts, q_lens, kv_lens, prev_ids)
            if self._steps_run % 32 == 0:
                ops.poll_status()
        else:
            fused = self._fused_blocks(B) if all_last else 0
            nsplits = [self._plan_splits(gi, q_lens, kv_lens, MAX_KV_SPLIT, fused_blocks=fused) for gi in range(len(self.mgr.groups))]
            max_splits = [max(ns) for ns in nsplits]
            self.last_plan = {"graph_key": None, "nsplits": nsplits, "max_split": max_splits}
            max_pages = [max(int(g.n_pages[e.slot]) for e in entries) for g in self.mgr.groups]
            lay = _Layout(T, B, len(want_rows), max_pages)
            host, idx = self._pinned_buffer(lay.size)
            self._fill(host.numpy(), lay, entries, starts, want_rows, nsplits)
            if self._dev_staging is None or self._dev_staging.numel() < lay.size:
                self._dev_staging = torch.empty(max(lay.size, 1 << 16), dtype=torch.int32, device=self.device)
            dev = self._dev_staging
            dev[:lay.size].copy_(host[:lay.size], non_blocking=True)
            self._mark(idx)
            self.last_h2d_bytes = 4 * lay.size
            if prev_ids is not None:
                ops.resolve_ids(dev[lay.input_ids: lay.input_ids + T], prev_ids)
            ctx = self._context(dev, lay, q_lens, kv_lens, [e.slot for e in entries], max_splits, uniform, nsplits,
                                all_rows_wanted=all_last)
            rows = dev[lay.want: lay.want + len(want_rows)]
            logits = self.model.forward(ctx, self._caches(ctx), rows)
            ops.poll_status()
        for e in entries:
            self.mgr.commit(e.slot, len(e.tokens))
        return logits

    def _mark(self, idx: int) -> None:
        ev = self._pinned_ev[idx]
        if ev is None:
            ev = self._pinned_ev[idx] = self._new_event()
        ev.record()

    # -- decode through CUDA graphs --------------------------------------------------------------
    @staticmethod
    def _bucket(b: int) -> int:
        """Captured batch sizes: 1, 2, 4, 8, then multiples of 16 (the reference's buckets,
        mini_sglang/managers/cuda_graph_runner.py:72-82)."""
        for c in (1, 2, 4, 8):
            if b <= c:
                return c
        return -(-b // 16) * 16

    def _graph_max_split(self, gi: int, b: int) -> int:
        n_kv, G, per_sm, _ = self._group_geom[gi]
        chunks = 1 if G <= 16 else -(-G // 16)
        blocks = b * n_kv * chunks
        places = self._fused_blocks(b) or self.sm_count * per_sm
        return max(1, min(MAX_KV_SPLIT, places // blocks))

    def _step_graph(self, entries, starts, q_lens, kv_lens, prev_ids=None) -> torch.Tensor:
        B = len(entries)
        b = self._bucket(B)
        need_pages = [max(int(g.n_pages[e.slot]) for e in entries) for g in self.mgr.groups]
        mp = tuple(max(8, 1 << (n - 1).bit_length()) for n in need_pages)
        # the graph fixes the launch's split dimension: the narrow one suits requests of like length; a batch
        # with a request far longer than the rest takes a second graph with room for more pieces
        room = [self._graph_max_split(gi, b) for gi in range(len(self.mgr.groups))]
        narrow = [min(c, MANY_SPLITS) for c in room]
        fused = self._fused_blocks(b)
        even_cuts = None
        if not fused and self._even_nb and self._wants_even_cut(kv_lens):
            # long contexts: the keys of all requests dealt out evenly over as many blocks as the SMs hold at once
            pieces = [min(EVEN_MAX_PIECES, nb) for nb in self._even_nb]
            even_cuts = [plan_even_cut(kv_lens, g.window, nb, mx) for g, nb, mx in zip(self.mgr.groups, self._even_nb, pieces)]
            nsplits = [c[5].tolist() for c in even_cuts]
            key = (b, mp, "even")
            gr = self._graphs.get(key)
            if gr is None:
                gr = self._capture(b, mp, pieces, even_nb=self._even_nb)
                self._graphs[key] = gr
        else:
            nsplits = [self._plan_splits(gi, q_lens, kv_lens, room[gi], max(narrow[gi], WIDE_KV_SPLIT), fused_blocks=fused)
                       for gi in range(len(self.mgr.groups))]
            # blocks of pieces that a request does not have leave at once, but they are launched: a graph with the split
            # dimension of long contexts (up to MAX_KV_SPLIT) is kept apart from the one that every other step replays
            wide = any(max(ns) > cap for ns, cap in zip(nsplits, narrow))
            key = (b, mp, wide)
            gr = self._graphs.get(key)
            if gr is None:
                gr = self._capture(b, mp, [max(c, r, WIDE_KV_SPLIT) for c, r in zip(narrow, room)] if wide else narrow)
                self._graphs[key] = gr
        self.last_plan = {"graph_key": key, "nsplits": nsplits, "max_split": list(gr.max_split),
                          "even_blocks": [c[0] for c in even_cuts] if even_cuts else None}
        lay = gr.layout
        if self.device_meta:
            self._meta_on_device(gr, entries, starts, nsplits, b, even_cuts)
        else:
            host, idx = self._pinned_buffer(lay.size)
            self._fill(host.numpy(), lay, entries, starts, list(range(b)), nsplits, even_cuts=even_cuts)
            gr.dev.copy_(host[:lay.size], non_blocking=True)
            self._mark(idx)
            self.last_h2d_bytes = 4 * lay.size
        if prev_ids is not None:
            ops.resolve_ids(gr.dev[lay.input_ids: lay.input_ids + B], prev_ids)
        gr.graph.replay()
        ops.LAUNCHES += gr.n_kernels
        return gr.logits[:B]

    def _wants_even_cut(self, kv_lens: Sequence[int]) -> bool:
        """Whether a decode step deals its keys out evenly (plan_even_cut) instead of cutting every request by itself:
        when the requests' lengths differ (the longest EVEN_UNEVEN times the mean or more) and a request has
        EVEN_FROM_UNITS units or more in the mean.  Requests of like length fill the SMs as well cut one by one, with
        fewer runs and pieces; below that mean a run of keys is so short that the fixed cost of the runs a block strings
        together outweighs what the even load gains."""
        if os.environ.get("MSGL_EVEN_CUT", "1") == "0":
            return False
        for g in self.mgr.groups:
            units = [-(-(min(k, g.window + 1) if g.window else k) // DECODE_UNIT_KEYS) for k in kv_lens]
            mean = sum(units) / len(units)
            if mean >= EVEN_FROM_UNITS and max(units) >= EVEN_UNEVEN * mean:
                return True
        return False

    def _meta_on_device(self, gr: "_Graph", entries, starts, nsplits, b: int, even_cuts=None) -> None:
        """The fields of a decode step that the captured graph reads, made on the device.  The host sends one small
        buffer: token id, slot and position of every request, its kv splits per cache group, and per group the table
        rows of the requests whose pages changed since the last such step (whole rows; a request gets a page every
        page_size tokens)."""
        lay, B, G = gr.layout, len(entries), len(self.mgr.groups)
        rows = [self.mgr.take_dirty_rows(gi) for gi in range(G)]
        n_delta = [1 + 3 * len(r) + sum(len(t) for _, t in r) for r in rows]
        n_even = [ops.even_cut_size(b, nb) if (nb and even_cuts is not None) else 0 for nb in lay.even_nb]
        size = (3 + G) * B + sum(_align4(n) for n in n_delta) + sum(_align4(n) for n in n_even)
        host_t, idx = self._pinned_buffer(size)
        host = host_t.numpy()
        host[0:B] = [e.tokens[0] for e in entries]
        host[B:2 * B] = [e.slot for e in entries]
        host[2 * B:3 * B] = starts
        off = 3 * B
        ns_off = []
        for gi in range(G):
            host[off:off + B] = nsplits[gi]
            ns_off.append(off)
            off += B
        d_off = []
        for gi in range(G):
            d_off.append(off)
            recs = rows[gi]
            host[off] = len(recs)
            at = off + 1 + 3 * len(recs)
            for k, (slot, table_row) in enumerate(recs):
                host[off + 1 + 3 * k: off + 4 + 3 * k] = (slot, len(table_row), at - off)
                host[at:at + len(table_row)] = table_row
                at += len(table_row)
            off += _align4(n_delta[gi])
        e_off = []
        for gi in range(G):
            e_off.append(off)
            if n_even[gi]:
                host[off:off + n_even[gi]] = pack_even_cut(even_cuts[gi], b, lay.even_nb[gi])
            off += _align4(n_even[gi])
        if self._dev_compact is None or self._dev_compact.numel() < size:
            self._dev_compact = torch.empty(max(size, 1 << 14), dtype=torch.int32, device=self.device)
        dev = self._dev_compact
        dev[:size].copy_(host_t[:size], non_blocking=True)
        self._mark(idx)
        self.last_h2d_bytes = 4 * size
        g0 = gr.dev
        for gi in range(G):
            if rows[gi]:
                ops.table_delta(dev[d_off[gi]: d_off[gi] + n_delta[gi]], len(rows[gi]), self.storage.tables[gi])
            mp = lay.max_pages[gi]
            ops.decode_meta(dev[0:B], dev[B:2 * B], dev[2 * B:3 * B], dev[ns_off[gi]:ns_off[gi] + B], B, b, self.storage.tables[gi],
                            self.page_size, mp, gi == 0,
                            input_ids=g0[lay.input_ids:], positions=g0[lay.positions:], token_req=g0[lay.token_req:],
                            q_start=g0[lay.q_start:], kv_len=g0[lay.kv_len:], slots=g0[lay.slots:],
                            out_loc=g0[lay.out_loc[gi]:], nsplit=g0[lay.nsplit[gi]:], block_table=g0[lay.table[gi]:],
                            order=g0[lay.order[gi]:], window=int(self.mgr.groups[gi].window or 0),
                            even_in=dev[e_off[gi]: e_off[gi] + n_even[gi]] if n_even[gi] else None,
                            even_out=g0[lay.even[gi]:] if n_even[gi] else None)

    def _capture(self, b: int, mp: Tuple[int, ...], max_split: Sequence[int], even_nb: Optional[Sequence[int]] = None) -> _Graph:
        gr = _Graph()
        lay = _Layout(b, b, b, mp, even_nb)
        gr.layout = lay
        gr.dev = torch.zeros(lay.size, dtype=torch.int32, device=self.device)
        gr.max_split = list(max_split)
        host = np.zeros(lay.size, dtype=np.int32)
        self._fill(host, lay, [], [], list(range(b)), [[1] * b for _ in self.mgr.groups])
        gr.dev.copy_(torch.from_numpy(host))
        ctx = self._context(gr.dev, lay, [1] * b, [1] * b, [0] * b, gr.max_split, True, all_rows_wanted=True)
        caches = self._caches(ctx)
        rows = gr.dev[lay.want: lay.want + b]
        # two eager runs size every scratch buffer outside the graph's private pool
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.model.forward(ctx, caches, rows)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        gr.graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES
        with torch.cuda.graph(gr.graph, pool=self._graph_pool):
            gr.logits = self.model.forward(ctx, caches, rows)
        gr.n_kernels = ops.LAUNCHES - before
        return gr
