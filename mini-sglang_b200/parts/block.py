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
    (mini_sglang/models/qwen3.py:162-178).  Roles: norms "input" and "post_mixer", "mixer", "feed_forward";
    what the checkpoint calls each of them below the layer's prefix comes from the layer description
    (`LayerSpec.names`).  Position encodings with equal parameters are one object shared by all layers."""

    def __init__(self, layer_spec, env: BuildEnv):
        super().__init__(None, layer_spec.prefix, env)
        at = layer_spec.part_prefix
        self.position = None
        if layer_spec.position is not None:
            self.position = env.shared(layer_spec.position, lambda: build_part(
                POSITION_ENCODINGS, "position encoding", layer_spec.position, layer_spec.prefix, env))
        self.norm_in = build_part(NORMS, "norm", layer_spec.norms["input"], at("input"), env)
        self.norm_post = build_part(NORMS, "norm", layer_spec.norms["post_mixer"], at("post_mixer"), env)
        self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, at("mixer"), env, position=self.position)
        self.ffn = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward, at("feed_forward"), env)

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

    def fused_decode_fields(self):
        """This arrangement is the one the whole-step decode kernel walks (norm, mixer, residual sum, norm, feed-forward,
        residual sum); it takes part if all four parts do."""
        parts = {"norm_in": self.norm_in.fused_decode_fields(), "mixer": self.mixer.fused_decode_fields(),
                 "norm_post": self.norm_post.fused_decode_fields(), "ffn": self.ffn.fused_decode_fields()}
        if any(v is None for v in parts.values()):
            return None
        return {"kind": "prenorm_residual", **parts}
