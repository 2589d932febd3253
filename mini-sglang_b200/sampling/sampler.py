from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import ops


class Sampler:
    """Greedy and temperature sampling on the device (one fused kernel per batch):
    argmax where temperature is 0, else an exponential race over softmax(logits / T), the rule
    of mini_sglang/layers/sampler.py:13-23.  The noise is a counter-based generator keyed by
    (seed, request key, request step), so a request's draws do not depend on the batch it is in."""

    def __init__(self, seed: int, device):
        self.seed = int(seed)
        self.device = device

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], row_keys: Sequence[int],
               steps: Sequence[int]) -> torch.Tensor:
        """-> int32 token ids [N] on the device."""
        if all(t == 0 for t in temperatures):
            return ops.sample(logits, None, None, None, self.seed)
        n = len(temperatures)
        host = torch.empty((3, n), dtype=torch.int32, pin_memory=True)
        host[0] = torch.tensor(list(temperatures), dtype=torch.float32).view(torch.int32)
        host[1] = torch.tensor([k & 0x7FFFFFFF for k in row_keys], dtype=torch.int32)
        host[2] = torch.tensor([s & 0x7FFFFFFF for s in steps], dtype=torch.int32)
        dev = host.to(self.device, non_blocking=True)
        return ops.sample(logits, dev[0].view(torch.float32), dev[1], dev[2], self.seed)
