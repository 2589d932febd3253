"""The model description every other part of the engine is built from.

A model is data: a list of layers, each naming its mixer, feed-forward, norms and position
encoding by registry key with their sizes and constants as parameters, and a run order
(`schedule`) that may name a layer twice or let a layer read another run's cache.  No part
reads config.json itself and no part knows which model it is in.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional


@dataclasses.dataclass(frozen=True)
class PartSpec:
    """A part chosen by registry key, with its sizes and constants."""

    kind: str
    params: Dict[str, Any] = dataclasses.field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclasses.dataclass
class LayerSpec:
    """One block: how the parts are arranged (`block`), and the parts themselves.

    `prefix` is the checkpoint name prefix of the layer's tensors ("model.layers.3"); `names` says what
    each part is called below it ("mixer" -> "self_attn" in a Qwen3 checkpoint)."""

    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]
    position: Optional[PartSpec] = None
    block: str = "prenorm_residual"
    # checkpoint sub-names of the layer's parts under `prefix`: the block's role -> the name the checkpoint uses
    # (roles "mixer", "feed_forward" and the keys of `norms`); a role that is not listed keeps its own name
    names: Dict[str, str] = dataclasses.field(default_factory=dict)

    def part_prefix(self, role: str) -> str:
        return f"{self.prefix}.{self.names.get(role, role)}"


@dataclasses.dataclass(frozen=True)
class Run:
    """One entry of the run order: run layer `layer` against cache `cache`.

    `cache` is an id chosen by the architecture; two runs with the same id share one cache.
    A run with `writes_cache=False` only reads what an earlier run wrote (its mixer computes
    no keys of its own).  `cache=None` means the mixer keeps nothing between steps."""

    layer: int
    cache: Optional[int] = None
    writes_cache: bool = True


@dataclasses.dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    layers: List[LayerSpec]
    schedule: List[Run]
    max_context_len: int
    eos_token_ids: List[int] = dataclasses.field(default_factory=list)
    checkpoint_dtype: str = "bfloat16"

    def validate(self) -> None:
        caches_written = set()
        for run in self.schedule:
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule names layer {run.layer}, the model has {len(self.layers)}")
            if run.cache is not None:
                if run.writes_cache:
                    caches_written.add(run.cache)
                elif run.cache not in caches_written:
                    raise ValueError(f"run of layer {run.layer} reads cache {run.cache} before any run wrote it")
