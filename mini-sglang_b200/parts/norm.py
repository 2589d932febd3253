from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """y = v * rsqrt(mean(v^2) + eps) * weight with v = residual + x, in float32; plain weight.
    Formula of mini_sglang/layers/layernorm.py:39-50.  params: size, eps, optional name
    (full tensor name; default "<prefix>.weight")."""

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.size, self.eps = int(spec["size"]), float(spec["eps"])
        self.tensor_name = spec.get("name") or self.name("weight")
        self.weight = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {self.tensor_name: TensorDecl((self.size,), kind="vector", init="norm")}

    def load(self, src) -> None:
        self.weight = src.fetch(self.tensor_name).contiguous()

    def forward(self, x=None, residual=None, residual_out=None, rows=None):
        return ops.rmsnorm(self.weight, self.eps, x=x, residual=residual, residual_out=residual_out, rows=rows,
                           out_dtype=self.env.dtype)

    def fused_decode_fields(self):
        return {"kind": "rmsnorm", "weight": self.weight, "eps": self.eps, "size": self.size}
