"""Interfaces and registries of the parts a model is assembled from.

A part is built from a PartSpec (its sizes and constants), the checkpoint-name prefix of the
layer it sits in, and a BuildEnv (activation dtype, device).  It declares the checkpoint
tensors it reads (`tensors`), takes them from a source (`load`), and computes (`forward`).
A part never sees config.json, the model's name, or any other part's internals.

    Mixer          forward(x [T, H], ctx, cache, writes_cache) -> [T, H]
                   cache_need() -> PagedKVNeed | StateNeed | None
    FeedForward    forward(x [T, H], ctx) -> [T, H]
    Norm           forward(x=None, residual=None, residual_out=None, rows=None) -> y
    PositionEncoding   rotary_table() -> float32 [max_pos, rot] or None;  apply(q, k, positions)
    Block          forward(delta, residual, ctx, cache, writes_cache) -> (delta, residual)

New kinds are added with the `register_*` decorators below; a model description then names
them by key.  The activations between parts are `env.dtype`; the residual stream is float32.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, Optional

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorDecl


@dataclasses.dataclass
class BuildEnv:
    dtype: torch.dtype
    device: torch.device
    _shared: Dict[Any, Any] = dataclasses.field(default_factory=dict, repr=False)

    def shared(self, spec: PartSpec, make: Callable[[], Any]):
        """One part per distinct (kind, parameters) among the parts that hold no checkpoint tensors of a
        layer's own (position encodings: 36 layers with the same rotation share one table)."""
        key = (spec.kind, tuple(sorted((k, repr(v)) for k, v in spec.params.items())))
        if key not in self._shared:
            self._shared[key] = make()
        return self._shared[key]


class Part:
    def __init__(self, spec: PartSpec, prefix: str, env: BuildEnv):
        self.spec, self.prefix, self.env = spec, prefix, env

    def name(self, suffix: str) -> str:
        return f"{self.prefix}.{suffix}" if self.prefix else suffix

    def tensors(self) -> Dict[str, TensorDecl]:
        return {}

    def load(self, src) -> None:
        pass

    def fused_decode_fields(self) -> Optional[Dict[str, Any]]:
        """What the whole-step decode kernel (csrc/decode_step.cu) needs of this part: its loaded tensors, sizes and
        constants under the names that kernel knows, or None if the part is of a kind the kernel does not compute
        (the default: a model with such a part is stepped kernel by kernel)."""
        return None


class Mixer(Part):
    # True if forward() only launches work whose shapes and addresses are fixed by (T, B) and reads
    # everything else (lengths, slots, tables) from the context's device tensors, so that a decode
    # step can be captured once and replayed.  Mixers that loop over requests on the host say False.
    graph_safe = False

    def cache_need(self):
        return None

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    # False if forward() reads device data on the host or launches work whose shapes depend on the
    # tokens (routing by gathered rows, say): a decode step with such a part is not captured in a CUDA graph.
    graph_safe = True

    def forward(self, x, ctx):
        raise NotImplementedError


class Norm(Part):
    def forward(self, x=None, residual=None, residual_out=None, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    """A position encoding that the attention mixer applies to q and k: a rotation of the first
    `rotary_dim` elements of every head (in halves or in neighbouring pairs, see `interleaved`) by angles that
    depend on the position and the element pair in any way the encoding likes.  (An encoding that is added to the hidden state instead
    belongs to an embedding part.)"""

    # which elements are rotated against each other: False: halves (element i with i + rotary_dim / 2, NeoX style);
    # True: neighbours (2 p with 2 p + 1, GPT-J style).  Pair p takes angle p of the table either way.
    interleaved = False

    def rotary_table(self) -> Optional[torch.Tensor]:
        """float32 [max_positions, rotary_dim] = cos | sin of the angles; rotary_dim may be smaller than
        the head size (partial rotation).  The fused q/k kernel applies it."""
        raise NotImplementedError


class Block(Part):
    def forward(self, delta, residual, ctx, cache, writes_cache: bool = True):
        raise NotImplementedError


MIXERS: Dict[str, Callable[..., Mixer]] = {}
FEED_FORWARDS: Dict[str, Callable[..., FeedForward]] = {}
NORMS: Dict[str, Callable[..., Norm]] = {}
POSITION_ENCODINGS: Dict[str, Callable[..., PositionEncoding]] = {}
BLOCKS: Dict[str, Callable[..., Block]] = {}
EMBEDDINGS: Dict[str, Callable[..., Part]] = {}
HEADS: Dict[str, Callable[..., Part]] = {}


def _register(table: Dict[str, Any], what: str):
    def deco_factory(kind: str):
        def deco(cls):
            table[kind] = cls
            return cls
        return deco
    deco_factory.__doc__ = f"Class decorator: make a {what} available to model descriptions under a key."
    return deco_factory


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_block = _register(BLOCKS, "block arrangement")
register_embedding = _register(EMBEDDINGS, "embedding")
register_head = _register(HEADS, "output head")


def build_part(table: Dict[str, Any], what: str, spec: PartSpec, prefix: str, env: BuildEnv, **kw):
    if spec.kind not in table:
        raise KeyError(f"unknown {what} {spec.kind!r}; registered: " + ", ".join(sorted(table)))
    return table[spec.kind](spec, prefix, env, **kw)
