from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import Part, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    """h = E[ids], no scaling (mini_sglang/layers/embed_head.py:49); the result opens the float32
    residual stream.  params: vocab_size, hidden_size, name.  An embedding part gets the step's context too
    (`ctx.positions` for one that adds a position's own vector); this one does not need it."""

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.V, self.H = int(spec["vocab_size"]), int(spec["hidden_size"])
        self.tensor_name = spec.get("name") or self.name("weight")
        self.weight = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {self.tensor_name: TensorDecl((self.V, self.H))}

    def load(self, src) -> None:
        self.weight = src.fetch(self.tensor_name).contiguous()

    def forward(self, ids: torch.Tensor, ctx=None) -> torch.Tensor:
        return ops.embedding(ids, self.weight)

    def fused_decode_fields(self):
        return {"kind": "token_embedding", "weight": self.weight, "V": self.V, "H": self.H}


@register_head("lm_head")
class LMHead(Part):
    """logits = h @ W^T in float32 output; W is the embedding matrix itself when tied
    (mini_sglang/models/qwen3.py:216-223, mini_sglang/layers/logits_processor.py:56-59).
    params: vocab_size, hidden_size, tied, name, tied_to."""

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.V, self.H = int(spec["vocab_size"]), int(spec["hidden_size"])
        self.tied = bool(spec.get("tied", False))
        self.tensor_name = spec.get("name") or self.name("weight")
        self.tied_to = spec.get("tied_to")
        self.weight = None

    def tensors(self) -> Dict[str, TensorDecl]:
        # a tied checkpoint may still carry a copy of the head; it is then ignored
        return {self.tensor_name: TensorDecl((self.V, self.H), optional=self.tied)}

    def load(self, src, embedding: TokenEmbedding = None) -> None:
        if self.tied:
            if embedding is None or embedding.tensor_name != self.tied_to:
                raise ValueError(f"tied head wants {self.tied_to!r}")
            self.weight = embedding.weight
        else:
            self.weight = src.fetch(self.tensor_name).contiguous()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return ops.linear(h, self.weight, out_dtype=torch.float32)

    def fused_decode_fields(self):
        return {"kind": "lm_head", "weight": self.weight, "V": self.V, "H": self.H}
