from __future__ import annotations

from typing import Dict

from ..weights.loader import TensorDecl
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, BuildEnv, build_part,
                   register_block)


@register_block("prenorm_residual")
class PreNormResidualBlock(Block):
    """res += delta_in; y = norm_in(res); a = mixer(y); res += a; y = norm_post(res); delta_out = ffn(y)

    The block returns its feed-forward output un-added together with the stream, so the next
    norm (the next block's, or the model's final norm) fuses the sum, as the reference does
    (mini_sglang/models/qwen3.py:162-178).  Norm names: "input" and "post_mixer", stored in the
    checkpoint as input_layernorm / post_attention_layernorm; mixer under self_attn, feed-forward
    under mlp."""

    NORM_NAMES = {"input": "input_layernorm", "post_mixer": "post_attention_layernorm"}

    def __init__(self, layer_spec, env: BuildEnv):
        super().__init__(None, layer_spec.prefix, env)
        p = layer_spec.prefix
        self.position = None
        if layer_spec.position is not None:
            self.position = build_part(POSITION_ENCODINGS, "position encoding", layer_spec.position, p, env)
        self.norm_in = build_part(NORMS, "norm", layer_spec.norms["input"], f"{p}.{self.NORM_NAMES['input']}", env)
        self.norm_post = build_part(NORMS, "norm", layer_spec.norms["post_mixer"], f"{p}.{self.NORM_NAMES['post_mixer']}", env)
        self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, f"{p}.self_attn", env, position=self.position)
        self.ffn = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward, f"{p}.mlp", env)

    def parts(self):
        return [p for p in (self.position, self.norm_in, self.mixer, self.norm_post, self.ffn) if p is not None]

    def tensors(self) -> Dict[str, TensorDecl]:
        out: Dict[str, TensorDecl] = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, src) -> None:
        for part in self.parts():
            part.load(src)

    def forward(self, delta, residual, ctx, cache, writes_cache: bool = True):
        # residual: float32 stream, updated in place; delta: the previous block's output or None
        y = self.norm_in.forward(x=delta, residual=residual, residual_out=residual if delta is not None else None)
        a = self.mixer.forward(y, ctx, cache, writes_cache)
        y = self.norm_post.forward(x=a, residual=residual, residual_out=residual)
        return self.ffn.forward(y, ctx), residual
