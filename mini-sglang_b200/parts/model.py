"""The model: embedding, the layers run in the order the description gives, final norm on the
rows whose logits are wanted, output head.

The reference's counterpart is mini_sglang/models/qwen3.py:181-236 (Qwen3Model.forward: embedding,
layers passing (hidden, residual), final norm; Qwen3ForCausalLM.forward: the head on the last row of
every request through mini_sglang/layers/logits_processor.py:47-67).  Here the layer list and its order
come from the ModelSpec, and the rows are whatever places the step asks for."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import ModelSpec
from ..weights.loader import TensorDecl
from .base import BLOCKS, EMBEDDINGS, HEADS, NORMS, BuildEnv, build_part
from .context import StepContext


NVTX_RANGES = False      # set by the engine's --profile: NVTX ranges around every run of a layer


class DecoderModel:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        self.spec, self.env = spec, env
        self.embedding = build_part(EMBEDDINGS, "embedding", spec.embedding, "", env)
        self.layers = []
        for ls in spec.layers:
            if ls.block not in BLOCKS:
                raise KeyError(f"unknown block arrangement {ls.block!r}; registered: " + ", ".join(sorted(BLOCKS)))
            self.layers.append(BLOCKS[ls.block](ls, env))
        self.final_norm = build_part(NORMS, "norm", spec.final_norm, "", env)
        self.head = build_part(HEADS, "output head", spec.head, "", env)
        self.schedule = list(spec.schedule)
        self.fused_decode = None

    # -- weights -----------------------------------------------------------------------
    def tensors(self) -> Dict[str, TensorDecl]:
        out: Dict[str, TensorDecl] = {}
        for part in [self.embedding, *self.layers, self.final_norm, self.head]:
            for name, decl in part.tensors().items():
                if name in out and out[name].shape != decl.shape:
                    raise ValueError(f"tensor {name!r} is declared twice with different shapes")
                out[name] = decl
        return out

    def load(self, src) -> None:
        self.embedding.load(src)
        for layer in self.layers:
            layer.load(src)
        self.final_norm.load(src)
        self.head.load(src, embedding=self.embedding)
        from .fused_decode import FusedDecodeStep
        self.fused_decode = FusedDecodeStep.build(self)      # None: this model is stepped kernel by kernel

    def cache_needs(self) -> Dict[int, object]:
        """cache id -> need, from the mixer of the run that writes the cache."""
        needs: Dict[int, object] = {}
        for run in self.schedule:
            if run.cache is None or not run.writes_cache:
                continue
            need = self.layers[run.layer].mixer.cache_need()
            if need is None:
                continue
            if run.cache in needs and needs[run.cache] != need:
                raise ValueError(f"cache {run.cache} is written by mixers with different needs")
            needs[run.cache] = need
        return needs

    # -- compute -----------------------------------------------------------------------
    def forward(self, ctx: StepContext, caches: Dict[int, object], want_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """-> float32 logits [len(want_rows), vocab] (all T rows if want_rows is None)."""
        if self.fused_decode is not None and self.fused_decode.takes(ctx):
            return self.fused_decode.forward(ctx, caches)       # the whole step in one persistent kernel
        if NVTX_RANGES:
            return self._forward_marked(ctx, caches, want_rows)
        residual = self.embedding.forward(ctx.input_ids, ctx)
        delta = None
        for run in self.schedule:
            cache = caches.get(run.cache) if run.cache is not None else None
            delta, residual = self.layers[run.layer].forward(delta, residual, ctx, cache, run.writes_cache)
        h = self.final_norm.forward(x=delta, residual=residual, rows=want_rows)
        return self.head.forward(h)

    def _forward_marked(self, ctx, caches, want_rows):
        """The same with an NVTX range around the embedding, every run of a layer and the head, for profilers
        that show them on the timeline."""
        nvtx = torch.cuda.nvtx
        nvtx.range_push("embedding")
        residual = self.embedding.forward(ctx.input_ids, ctx)
        nvtx.range_pop()
        delta = None
        for i, run in enumerate(self.schedule):
            nvtx.range_push(f"run {i}: layer {run.layer}")
            cache = caches.get(run.cache) if run.cache is not None else None
            delta, residual = self.layers[run.layer].forward(delta, residual, ctx, cache, run.writes_cache)
            nvtx.range_pop()
        nvtx.range_push("final norm + head")
        h = self.final_norm.forward(x=delta, residual=residual, rows=want_rows)
        out = self.head.forward(h)
        nvtx.range_pop()
        return out


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorDecl]:
    """The checkpoint tensors of a model description, without touching a device."""
    env = BuildEnv(dtype=torch.bfloat16, device=torch.device("cpu"))
    return DecoderModel(spec, env).tensors()
