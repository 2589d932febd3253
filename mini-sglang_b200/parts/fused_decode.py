"""The whole decode step of a few requests as ONE persistent kernel (csrc/decode_step.cu).

A model takes this path when every part of it says it can (`Part.fused_decode_fields`): token embedding, blocks of
the pre-norm residual arrangement with RMSNorm, paged attention over all keys (per-head q/k norm and a rotary table
optional) and a SwiGLU feed-forward, RMSNorm and a linear head; all layers of the same sizes, every run of the
schedule writing a cache of its own; bfloat16.  Anything else is stepped kernel by kernel as before, and so is every
step that is not "one new token for each of at most FUSED_DECODE_MAX_TOKENS requests, all logits wanted".  The
reference has no counterpart: its decode step is the same module-by-module forward as its prefill
(mini_sglang/models/qwen3.py:181-236) replayed from a CUDA graph.

The kernel gets the layers as an array of pointer records in device memory, written once per set of caches.
"""

from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

import torch

from .. import ops
from .context import KVCacheView, StepContext


def _same(values) -> bool:
    values = list(values)
    return all(v == values[0] for v in values[1:])


class FusedDecodeStep:
    @classmethod
    def build(cls, model) -> Optional["FusedDecodeStep"]:
        """-> the fused step of `model` (a DecoderModel with its tensors loaded), or None if it does not qualify."""
        if not ops.USE_FUSED_DECODE or model.env.dtype != torch.bfloat16 or model.env.device.type != "cuda":
            return None
        emb, fin, head = model.embedding.fused_decode_fields(), model.final_norm.fused_decode_fields(), model.head.fused_decode_fields()
        blocks = [b.fused_decode_fields() for b in model.layers]
        if emb is None or fin is None or head is None or not blocks or any(b is None for b in blocks):
            return None
        if emb["kind"] != "token_embedding" or fin["kind"] != "rmsnorm" or head["kind"] != "lm_head":
            return None
        for b in blocks:
            kinds = (b["kind"], b["norm_in"]["kind"], b["mixer"]["kind"], b["norm_post"]["kind"], b["ffn"]["kind"])
            if kinds != ("prenorm_residual", "rmsnorm", "paged_attention", "rmsnorm", "swiglu_mlp"):
                return None
        mix, ffn = [b["mixer"] for b in blocks], [b["ffn"] for b in blocks]
        for key in ("H", "n_q", "n_kv", "d", "scale"):
            if not _same(m[key] for m in mix):
                return None
        if not _same(f["I"] for f in ffn) or not _same(f["H"] for f in ffn) or ffn[0]["H"] != mix[0]["H"]:
            return None
        H, V = mix[0]["H"], head["V"]
        if emb["H"] != H or head["H"] != H or fin["size"] != H or emb["V"] != V:
            return None
        ropes = [m["rope"] for m in mix]
        if any((r is None) != (ropes[0] is None) for r in ropes):
            return None
        if ropes[0] is not None and not all(r["table"].data_ptr() == ropes[0]["table"].data_ptr() for r in ropes):
            return None
        if not _same((m["q_norm"] is None, m["k_norm"] is None) for m in mix) or (mix[0]["q_norm"] is None) != (mix[0]["k_norm"] is None):
            return None
        # norm weights of one element type throughout (a checkpoint keeps them all alike)
        nws = [b["norm_in"]["weight"] for b in blocks] + [b["norm_post"]["weight"] for b in blocks]
        if not _same(w.dtype for w in nws) or nws[0].dtype not in (torch.float32, torch.bfloat16):
            return None
        if mix[0]["q_norm"] is not None and not _same(m["q_norm"].dtype for m in mix):
            return None
        for t in [emb["weight"], head["weight"]] + [m["qkv"] for m in mix] + [m["o"] for m in mix] + \
                 [f["gate_up"] for f in ffn] + [f["down"] for f in ffn]:
            if t.dtype != torch.bfloat16 or not t.is_contiguous() or t.data_ptr() % 16:
                return None
        # every run of the schedule with a cache of its own that it writes
        seen = set()
        for run in model.schedule:
            if run.cache is None or not run.writes_cache or run.cache in seen:
                return None
            seen.add(run.cache)
        sizes = dict(H=H, n_q=mix[0]["n_q"], n_kv=mix[0]["n_kv"], d=mix[0]["d"], I=ffn[0]["I"], V=V)
        if ops.decode_step_blocks(1, H, sizes["n_q"], sizes["n_kv"], sizes["d"], sizes["I"], V) <= 0:
            return None
        return cls(model, blocks, emb, fin, head, sizes)

    def __init__(self, model, blocks, emb, fin, head, sizes):
        self.model, self.blocks, self.emb, self.fin, self.head = model, blocks, emb, fin, head
        self.H, self.n_q, self.n_kv, self.d, self.I, self.V = (sizes[k] for k in ("H", "n_q", "n_kv", "d", "I", "V"))
        self.scale = float(blocks[0]["mixer"]["scale"])
        self.rope = blocks[0]["mixer"]["rope"]
        self.device = model.env.device
        self._layer_arrays: Dict[tuple, torch.Tensor] = {}        # by the caches' addresses
        self._bar = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._tickets = torch.zeros(ops.FUSED_DECODE_MAX_TOKENS * self.n_kv, dtype=torch.int32, device=self.device)
        self._blocks: Dict[int, int] = {}

    def blocks_for(self, tokens: int) -> int:
        """Blocks of the kernel's launch for a step of `tokens` requests (what the kv splits are planned against)."""
        if tokens not in self._blocks:
            self._blocks[tokens] = ops.decode_step_blocks(tokens, self.H, self.n_q, self.n_kv, self.d, self.I, self.V)
        return self._blocks[tokens]

    def takes(self, ctx: StepContext) -> bool:
        return (ctx.uniform_decode and ctx.all_rows_wanted and 0 < ctx.B <= ops.FUSED_DECODE_MAX_TOKENS
                and len(ctx.groups) == 1 and ctx.groups[0].window is None and self.blocks_for(ctx.B) > 0)

    def _layers_on_device(self, caches: Dict[int, object]) -> torch.Tensor:
        runs = self.model.schedule
        views: List[KVCacheView] = [caches[run.cache] for run in runs]
        key = tuple((v.k.data_ptr(), v.v.data_ptr()) for v in views)
        arr = self._layer_arrays.get(key)
        if arr is not None:
            return arr
        recs = (ops.DsLayer * len(runs))()
        for rec, run, view in zip(recs, runs, views):
            b = self.blocks[run.layer]
            m, f = b["mixer"], b["ffn"]
            if view.k.dtype != torch.bfloat16 or not view.k.is_contiguous() or not view.v.is_contiguous():
                raise ops.KernelError("decode_step: the cache must be contiguous bfloat16")
            rec.w_qkv, rec.b_qkv, rec.w_o = m["qkv"].data_ptr(), ops._ptr(m["qkv_bias"]), m["o"].data_ptr()
            rec.w_gu, rec.w_down = f["gate_up"].data_ptr(), f["down"].data_ptr()
            rec.norm_in, rec.norm_post = b["norm_in"]["weight"].data_ptr(), b["norm_post"]["weight"].data_ptr()
            rec.q_norm, rec.k_norm = ops._ptr(m["q_norm"]), ops._ptr(m["k_norm"])
            rec.k_cache, rec.v_cache = view.k.data_ptr(), view.v.data_ptr()
            rec.eps_in, rec.eps_post, rec.eps_qk = b["norm_in"]["eps"], b["norm_post"]["eps"], m["qk_norm_eps"]
            rec.norm_f32 = int(b["norm_in"]["weight"].dtype == torch.float32)
            rec.qk_norm_f32 = int(m["q_norm"] is not None and m["q_norm"].dtype == torch.float32)
        raw = bytes(recs)
        arr = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(self.device)
        self._layer_arrays[key] = arr
        return arr

    def prepare(self, caches: Dict[int, object]) -> None:
        """Everything that allocates or copies, done ahead of a stream capture."""
        self._layers_on_device(caches)
        ops._status_tensor(self.device)

    def forward(self, ctx: StepContext, caches: Dict[int, object]) -> torch.Tensor:
        """-> float32 logits [B, vocab] of the step's B tokens."""
        g = ctx.groups[0]
        B, ws = ctx.B, ctx.workspace
        layers = self._layers_on_device(caches)
        max_split = g.max_split if g.nsplit is not None else 1
        M8 = ops.FUSED_DECODE_MAX_TOKENS
        qkv_n = (self.n_q + 2 * self.n_kv) * self.d
        res = ws.get("ds_res", M8 * self.H, torch.float32)
        xn = ws.get("ds_xn", M8 * self.H, torch.bfloat16)
        ssq = ws.get("ds_ssq", 8 * max(self.blocks_for(B), 1), torch.float32)
        qkv = ws.get("ds_qkv", M8 * qkv_n, torch.bfloat16)
        attn = ws.get("ds_attn", M8 * self.n_q * self.d, torch.bfloat16)
        act = ws.get("ds_act", M8 * self.I, torch.bfloat16)
        part_o = ws.get("attn_part_o", max(max_split, 1) * M8 * self.n_q * self.d, torch.float32)
        part_ml = ws.get("attn_part_ml", max(max_split, 1) * M8 * self.n_q * 2, torch.float32)
        logits = torch.empty((B, self.V), dtype=torch.float32, device=self.device)
        page = ctx.page_size
        st = ops.DsStep()
        st.layers, st.n_layers, st.M = layers.data_ptr(), len(self.model.schedule), B
        st.H, st.n_q, st.n_kv, st.I, st.V = self.H, self.n_q, self.n_kv, self.I, self.V
        st.page_size = page
        st.page_shift = page.bit_length() - 1 if page & (page - 1) == 0 else -1
        st.bt_stride, st.max_split, st.scale = g.block_table.stride(0), max_split, self.scale
        if self.rope is not None:
            st.rope, st.rot, st.max_pos = self.rope["table"].data_ptr(), self.rope["rot"], self.rope["table"].shape[0]
        st.ids, st.positions, st.kv_len = ctx.input_ids.data_ptr(), ctx.positions.data_ptr(), ctx.kv_len.data_ptr()
        st.block_table, st.out_loc, st.nsplit = g.block_table.data_ptr(), g.out_loc.data_ptr(), ops._ptr(g.nsplit)
        st.embed, st.final_norm = self.emb["weight"].data_ptr(), self.fin["weight"].data_ptr()
        st.final_f32, st.eps_final = int(self.fin["weight"].dtype == torch.float32), self.fin["eps"]
        st.lm_head = self.head["weight"].data_ptr()
        st.res, st.qkv, st.attn, st.act = res.data_ptr(), qkv.data_ptr(), attn.data_ptr(), act.data_ptr()
        st.xn, st.ssq = xn.data_ptr(), ssq.data_ptr()
        st.part_o, st.part_ml, st.tickets, st.logits = part_o.data_ptr(), part_ml.data_ptr(), self._tickets.data_ptr(), logits.data_ptr()
        st.bar = self._bar.data_ptr()
        st.status = ops._status_tensor(self.device).data_ptr() + 4 * ops.STATUS_WORD_DECODE_STEP
        ops.decode_step(st, self.d)
        return logits
