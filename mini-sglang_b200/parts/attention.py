from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..cache.manager import PagedKVNeed
from ..weights.loader import TensorDecl
from .base import Mixer, register_mixer
from .context import KVCacheView, StepContext


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    """Causal grouped-query attention over the paged cache.

    qkv = x Wqkv^T (+ b); optional per-head RMSNorm of q and k (one weight of head size shared by
    all heads, before the rotation); rotary position encoding; k and v written to the cache before
    attention so the new tokens read themselves from it; softmax(scale * q K^T) V with query head h
    on kv head h // (n_q / n_kv); output projection.  Order and formulas:
    mini_sglang/models/qwen3.py:86-97, mini_sglang/layers/attn/fa3_attn_backend.py:94-117.
    q_proj/k_proj/v_proj are packed row-wise as [q; k; v] (mini_sglang/layers/linear.py:182-205).

    params: hidden_size, num_heads, num_kv_heads, head_dim, scale, qkv_bias, qk_norm, qk_norm_eps,
            window (None = all keys; W = the last W keys).
    """

    graph_safe = True

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        s = spec
        self.H, self.n_q, self.n_kv, self.d = int(s["hidden_size"]), int(s["num_heads"]), int(s["num_kv_heads"]), int(s["head_dim"])
        if self.n_q % self.n_kv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.scale = float(s.get("scale", self.d ** -0.5))
        self.qkv_bias = bool(s.get("qkv_bias", False))
        self.qk_norm = bool(s.get("qk_norm", False))
        self.qk_norm_eps = float(s.get("qk_norm_eps", 1e-6))
        self.window = s.get("window")
        self.position = position
        self.use_mma = ops.mma_supported(self.d, env.dtype)
        if self.d > 512:
            raise ValueError(f"head size {self.d}: the attention kernels take head sizes up to 512")
        self.qkv = self.qkv_b = self.o = self.q_norm = self.k_norm = None

    # -- weights -----------------------------------------------------------------------
    def tensors(self) -> Dict[str, TensorDecl]:
        qd, kd = self.n_q * self.d, self.n_kv * self.d
        t = {self.name("q_proj.weight"): TensorDecl((qd, self.H)),
             self.name("k_proj.weight"): TensorDecl((kd, self.H)),
             self.name("v_proj.weight"): TensorDecl((kd, self.H)),
             self.name("o_proj.weight"): TensorDecl((self.H, qd))}
        if self.qkv_bias:
            t[self.name("q_proj.bias")] = TensorDecl((qd,), kind="vector")
            t[self.name("k_proj.bias")] = TensorDecl((kd,), kind="vector")
            t[self.name("v_proj.bias")] = TensorDecl((kd,), kind="vector")
        if self.qk_norm:
            t[self.name("q_norm.weight")] = TensorDecl((self.d,), kind="vector", init="norm")
            t[self.name("k_norm.weight")] = TensorDecl((self.d,), kind="vector", init="norm")
        return t

    def load(self, src) -> None:
        f = src.fetch
        self.qkv = torch.cat((f(self.name("q_proj.weight")), f(self.name("k_proj.weight")),
                              f(self.name("v_proj.weight"))), dim=0).contiguous()
        self.o = f(self.name("o_proj.weight")).contiguous()
        if self.qkv_bias:
            self.qkv_b = torch.cat((f(self.name("q_proj.bias")), f(self.name("k_proj.bias")),
                                    f(self.name("v_proj.bias"))), dim=0).to(self.env.dtype).contiguous()
        if self.qk_norm:
            self.q_norm = f(self.name("q_norm.weight")).contiguous()
            self.k_norm = f(self.name("k_norm.weight")).to(self.q_norm.dtype).contiguous()

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(self.n_kv, self.d, self.window, q_heads=self.n_q)

    def fused_decode_fields(self):
        if self.window is not None or (self.position is not None and (self.position.fused_decode_fields() is None
                                                                      or self.position.interleaved)):
            return None
        rope = self.position.fused_decode_fields() if self.position is not None else None
        return {"kind": "paged_attention", "qkv": self.qkv, "qkv_bias": self.qkv_b, "o": self.o, "q_norm": self.q_norm,
                "k_norm": self.k_norm, "qk_norm_eps": self.qk_norm_eps, "H": self.H, "n_q": self.n_q, "n_kv": self.n_kv,
                "d": self.d, "scale": self.scale, "rope": rope}

    # -- compute -----------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: KVCacheView, writes_cache: bool = True) -> torch.Tensor:
        qkv = ops.linear(x, self.qkv, self.qkv_b)
        table = self.position.rotary_table() if self.position is not None else None
        q = ops.qknorm_rope_kvwrite(
            qkv, ctx.positions, self.n_q, self.n_kv, self.d,
            q_weight=self.q_norm, k_weight=self.k_norm, eps=self.qk_norm_eps, rope_table=table,
            out_loc=cache.group.out_loc if writes_cache else None,
            k_cache=cache.k if writes_cache else None, v_cache=cache.v if writes_cache else None,
            page_size=cache.page_size, interleaved=bool(getattr(self.position, "interleaved", False)))
        out = torch.empty_like(q)
        self.attend(q, out, ctx, cache)
        return ops.linear(out.view(ctx.T, self.n_q * self.d), self.o)

    def attend(self, q: torch.Tensor, out: torch.Tensor, ctx: StepContext, cache: KVCacheView) -> None:
        g = cache.group
        G = self.n_q // self.n_kv
        window = int(self.window or 0)
        max_split = g.max_split if g.nsplit is not None else 1
        part_o = part_ml = None
        if max_split > 1:
            rows = max_split * ctx.T * self.n_q
            part_o = ctx.workspace.get("attn_part_o", rows * self.d, torch.float32)
            part_ml = ctx.workspace.get("attn_part_ml", rows * 2, torch.float32)
        common = dict(q_start=ctx.q_start, kv_len=ctx.kv_len, block_table=g.block_table,
                      nsplit=g.nsplit if max_split > 1 else None, part_o=part_o, part_ml=part_ml, n_kv=self.n_kv,
                      page_size=cache.page_size, window=window, max_split=max_split, scale=self.scale,
                      uniform_decode=ctx.uniform_decode, order=g.order if ctx.uniform_decode else None)
        big = 1 << 30
        if not self.use_mma:
            qt = ops.attention_tile_tokens(ops.VARIANT_SIMT, G)
            gx = ctx.B if ctx.uniform_decode else sum(-(-n // qt) for n in ctx.host_q_lens)
            ops.attention(q, out, cache.k, cache.v, qlen_min=1, qlen_max=big, variant=ops.VARIANT_SIMT, grid_x=gx, **common)
        else:
            qt_dec = ops.attention_tile_tokens(ops.VARIANT_MMA_DECODE, G, self.d)
            qt_row = ops.attention_tile_tokens(ops.VARIANT_MMA_ROWS, G)
            if ctx.uniform_decode:
                ops.attention(q, out, cache.k, cache.v, qlen_min=1, qlen_max=1, variant=ops.VARIANT_MMA_DECODE,
                              grid_x=ctx.B, even=g.even, even_nb=g.even_nb, **common)
            else:
                n_dec = sum(1 for n in ctx.host_q_lens if n <= qt_dec)
                n_row = sum(-(-n // qt_row) for n in ctx.host_q_lens if n > qt_dec)
                if n_dec:
                    ops.attention(q, out, cache.k, cache.v, qlen_min=1, qlen_max=qt_dec,
                                  variant=ops.VARIANT_MMA_DECODE, grid_x=n_dec, **common)
                # the tcgen05 kernels take whole key ranges: only if no longer request has kv splits
                unsplit = max_split == 1 or (g.host_nsplit is not None and
                                             all(ns == 1 for n, ns in zip(ctx.host_q_lens, g.host_nsplit) if n > qt_dec))
                if n_row and unsplit and ops.tc_supported(self.d, q.dtype, G):
                    ops.attention_tc(q, out, cache.k, cache.v, q_start=ctx.q_start, kv_len=ctx.kv_len,
                                     block_table=g.block_table, n_kv=self.n_kv, page_size=cache.page_size, window=window,
                                     scale=self.scale, qlen_min=qt_dec + 1, qlen_max=big, q_lens=ctx.host_q_lens)
                elif n_row:
                    ops.attention(q, out, cache.k, cache.v, qlen_min=qt_dec + 1, qlen_max=big,
                                  variant=ops.VARIANT_MMA_ROWS, grid_x=n_row, **common)
        if max_split > 1:
            ops.attention_combine(part_o, part_ml, None if ctx.uniform_decode else ctx.token_req, g.nsplit, out, max_split)
