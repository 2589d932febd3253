"""Weights by tensor name.

A model's parts declare the checkpoint tensors they read (name, shape, kind).  `check_index`
compares that list with what a folder holds and raises ONE error naming every missing tensor,
every unexpected tensor and every wrong shape.  Sources hand tensors to the parts:
`CheckpointSource` reads a folder of safetensors, `RandomSource` draws seeded random values
(on the device for full-size benchmarks, on the CPU for writing a model folder).

Kept precision: bfloat16 stays bfloat16; integer tables become int32; a float tensor stored in
32 bits stays 32-bit unless it is a matrix operand of the bfloat16 GEMMs (which only take
bfloat16).  With compute dtype float32 every float tensor is widened to float32 (exact).
The reference loads by parameter name through per-parameter loaders
(mini_sglang/models/qwen3.py:238-261, mini_sglang/utils/loader.py:13-25) and does not notice
missing tensors; this loader does.
"""

from __future__ import annotations

import dataclasses
import hashlib
from typing import Dict, List, Optional, Tuple

import torch

from .safetensors_io import TensorEntry, open_model_dir


class WeightsError(ValueError):
    pass


@dataclasses.dataclass(frozen=True)
class TensorDecl:
    """A checkpoint tensor a part reads.  kind: "matrix" (GEMM / gather operand), "vector" (norm
    weights, biases), "int" (integer table).  init: how the random-weights mode fills it."""

    shape: Tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"          # "normal": N(0, std)   "norm": 1 + N(0, 0.05)   "zeros"
    optional: bool = False        # may be present and is then ignored (e.g. the head of a tied model)


def check_index(expected: Dict[str, TensorDecl], index: Dict[str, TensorEntry], where: str) -> None:
    missing = [n for n, d in expected.items() if not d.optional and n not in index]
    unexpected = [n for n in index if n not in expected]
    wrong = [(n, tuple(index[n].shape), tuple(d.shape)) for n, d in expected.items()
             if n in index and not d.optional and tuple(index[n].shape) != tuple(d.shape)]
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: the tensors do not match the model described by config.json"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " +
                     ", ".join(f"{n} is {list(a)}, expected {list(b)}" for n, a, b in sorted(wrong)))
    raise WeightsError("\n".join(lines))


def kept_dtype(stored: torch.dtype, kind: str, compute: torch.dtype) -> torch.dtype:
    if kind == "int" or not stored.is_floating_point:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if stored == torch.float32 and kind != "matrix":
        return torch.float32
    return torch.bfloat16


class CheckpointSource:
    def __init__(self, model_dir: str, expected: Dict[str, TensorDecl], compute_dtype: torch.dtype, device):
        self.files, self.index = open_model_dir(model_dir)
        check_index(expected, self.index, model_dir)
        self.expected, self.compute_dtype, self.device = expected, compute_dtype, device

    def has(self, name: str) -> bool:
        return name in self.index

    def fetch(self, name: str) -> torch.Tensor:
        e = self.index[name]
        decl = self.expected[name]
        t = e.file.read(name)
        return t.to(device=self.device, dtype=kept_dtype(e.dtype, decl.kind, self.compute_dtype), copy=True)

    def close(self):
        for f in self.files:
            f.close()


class RandomSource:
    """Seeded random tensors: matrices N(0, std), norm weights 1 + N(0, 0.05); each tensor has a
    generator of its own seeded by (seed, name), so the values do not depend on the order of
    the requests for them.  Values are drawn in float32 and rounded to `store_dtype`."""

    def __init__(self, expected: Dict[str, TensorDecl], seed: int, compute_dtype: torch.dtype, device,
                 store_dtype: torch.dtype = torch.bfloat16, std: float = 0.02):
        self.expected, self.seed, self.compute_dtype, self.device = expected, seed, compute_dtype, torch.device(device)
        self.store_dtype, self.std = store_dtype, std

    def has(self, name: str) -> bool:
        return name in self.expected and not self.expected[name].optional

    def draw(self, name: str) -> torch.Tensor:
        decl = self.expected[name]
        h = hashlib.sha256(f"{self.seed}:{name}".encode()).digest()
        g = torch.Generator(device=self.device).manual_seed(int.from_bytes(h[:7], "little"))
        if decl.kind == "int" or decl.init == "zeros":
            return torch.zeros(decl.shape, dtype=torch.int32 if decl.kind == "int" else self.store_dtype,
                               device=self.device)
        t = torch.randn(decl.shape, generator=g, dtype=torch.float32, device=self.device)
        t = 1.0 + 0.05 * t if decl.init == "norm" else self.std * t
        return t.to(self.store_dtype)

    def fetch(self, name: str) -> torch.Tensor:
        t = self.draw(name)
        return t.to(dtype=kept_dtype(t.dtype, self.expected[name].kind, self.compute_dtype))

    def close(self):
        pass
