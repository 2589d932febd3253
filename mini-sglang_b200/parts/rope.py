from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rope_neox")
class RotaryNeox(PositionEncoding):
    """Rotary position encoding, NeoX style: inv_freq_i = theta^(-2i/rot), angle = pos * inv_freq_i
    in float32, the two halves of the first `rotary_dim` elements rotated against each other.
    Table [max_positions, rotary_dim] = cos | sin in float32, as
    mini_sglang/layers/rotary_embedding.py:59-67 builds it; no scaling of any kind.
    params: head_dim, rotary_dim, theta, max_positions."""

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        self.theta = float(spec["theta"])
        self.max_positions = int(spec["max_positions"])
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self._table: Optional[torch.Tensor] = None

    def load(self, src) -> None:
        self.rotary_table()      # made with the weights, so that the memory left for the cache is measured after it

    def rotary_table(self) -> torch.Tensor:
        if self._table is None:
            # built on the host in float32, operation by operation as the reference does, so the
            # table does not depend on the device's pow/sin/cos roundings; then moved to the device
            idx = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
            inv_freq = 1.0 / (self.theta ** (idx / self.rotary_dim))
            t = torch.arange(self.max_positions, dtype=torch.float32)
            freqs = t[:, None] * inv_freq[None, :]
            self._table = torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous().to(self.env.device)
        return self._table

    def fused_decode_fields(self):
        return {"kind": "rotary_table", "table": self.rotary_table(), "rot": self.rotary_dim, "max_pos": self.max_positions}
