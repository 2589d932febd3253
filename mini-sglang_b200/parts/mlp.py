from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, register_feed_forward


@register_feed_forward("swiglu_mlp")
class SwiGLUMLP(FeedForward):
    """down(silu(gate(x)) * up(x)), dense, no biases (mini_sglang/models/qwen3.py:100-126).
    gate_proj and up_proj are packed row-wise into one [2I, H] matrix so one product feeds the
    activation kernel (the packing of mini_sglang/layers/linear.py:126-138).
    params: hidden_size, intermediate_size."""

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.H, self.I = int(spec["hidden_size"]), int(spec["intermediate_size"])
        self.gate_up = self.down = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {self.name("gate_proj.weight"): TensorDecl((self.I, self.H)),
                self.name("up_proj.weight"): TensorDecl((self.I, self.H)),
                self.name("down_proj.weight"): TensorDecl((self.H, self.I))}

    def load(self, src) -> None:
        self.gate_up = torch.cat((src.fetch(self.name("gate_proj.weight")), src.fetch(self.name("up_proj.weight"))),
                                 dim=0).contiguous()
        self.down = src.fetch(self.name("down_proj.weight")).contiguous()

    def forward(self, x, ctx):
        return ops.linear(ops.linear_swiglu(x, self.gate_up), self.down)

    def fused_decode_fields(self):
        return {"kind": "swiglu_mlp", "gate_up": self.gate_up, "down": self.down, "H": self.H, "I": self.I}
