from __future__ import annotations

import dataclasses
from typing import Any, Dict, Optional


@dataclasses.dataclass
class SamplingParams:
    """Names, meanings and defaults of mini_sglang/managers/sampling_params.py:4-19.
    temperature 0 is greedy; eos_token_id -1 means "the model's own end tokens"; `seed` (ours)
    fixes the noise of temperature sampling for the request."""

    temperature: float = 0.0
    max_new_tokens: int = 64
    ignore_eos: bool = False
    eos_token_id: int = -1
    seed: Optional[int] = None

    @classmethod
    def init_from_dict(cls, d: Optional[Dict[str, Any]]) -> "SamplingParams":
        d = dict(d or {})
        known = {f.name for f in dataclasses.fields(cls)}
        extra = set(d) - known
        if extra:
            raise ValueError(f"unknown sampling parameters {sorted(extra)}; known: {sorted(known)}")
        p = cls(**d)
        if p.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if p.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        return p
