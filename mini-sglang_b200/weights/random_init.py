"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.  The reference's `--dummy_load` fills parameters in memory with
N(0, 0.1) (mini_sglang/utils/loader.py:28-34); here the values go to disk under their
checkpoint names so that every consumer (this engine in either precision, a plain
implementation) reads the same numbers."""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Union

import torch

from ..config import architecture_of
from .loader import RandomSource
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


def write_random_model(model_dir: str, config: Union[Dict[str, Any], Any], seed: int, dtype: str = "bfloat16",
                       std: float = 0.02) -> str:
    """`config` is the content of a config.json (a dict with `architectures`) or a typed
    configuration with `to_dict()`."""
    from ..parts.model import expected_tensors

    raw = config if isinstance(config, dict) else config.to_dict()
    arch = architecture_of(raw)
    cfg = arch.config_cls.from_dict(raw)
    spec = arch.build_spec(cfg)
    spec.validate()
    expected = expected_tensors(spec)
    src = RandomSource(expected, seed, compute_dtype=torch.bfloat16, device="cpu", store_dtype=_STORE[dtype], std=std)
    os.makedirs(model_dir, exist_ok=True)
    out = dict(raw)
    out["torch_dtype"] = "bfloat16" if _STORE[dtype] == torch.bfloat16 else "float32"
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(out, f, indent=1)
    names = sorted(n for n, d in expected.items() if not d.optional)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), [(n, src.draw(n)) for n in names],
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir
