"""Qwen3 dense decoder: typed configuration and its model description.

Keys and defaults follow jason-fxz/mini-sglang: mini_sglang/utils/model_config.py:14-22
(sizes, max_position_embeddings, torch_dtype) and mini_sglang/models/qwen3.py:138-152,216
(rms_norm_eps, attention_bias default False, head_dim default hidden/heads, rope_theta
default 1e6, intermediate_size, hidden_act must be "silu", tie_word_embeddings).
"""

from __future__ import annotations

import dataclasses
from typing import Any, Dict, List

from .registry import ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, Run


@dataclasses.dataclass
class Qwen3Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    attention_bias: bool
    hidden_act: str
    torch_dtype: str
    eos_token_ids: List[int]

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen3Config":
        def need(key):
            if key not in raw or raw[key] is None:
                raise ConfigError(f"config.json: missing key {key!r}")
            return raw[key]

        n_q = int(need("num_attention_heads"))
        hidden = int(need("hidden_size"))
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if hidden % n_q:
                raise ConfigError("config.json: no head_dim and hidden_size is not a multiple of num_attention_heads")
            head_dim = hidden // n_q
        rope_theta = raw.get("rope_theta")
        if rope_theta is None:
            rope_theta = (raw.get("rope_parameters") or {}).get("rope_theta", 1000000.0)
        scaling = raw.get("rope_scaling") or (raw.get("rope_parameters") or {}).get("rope_type")
        if scaling not in (None, "default") and not (isinstance(scaling, dict) and scaling.get("rope_type", scaling.get("type")) in (None, "default")):
            raise ConfigError(f"config.json: rope scaling {scaling!r} is not part of this architecture")
        if raw.get("use_sliding_window", False):
            raise ConfigError("config.json: use_sliding_window=true is not part of this architecture")
        eos = raw.get("eos_token_id", [])
        eos = [] if eos is None else ([int(e) for e in eos] if isinstance(eos, (list, tuple)) else [int(eos)])
        cfg = cls(
            hidden_size=hidden,
            num_hidden_layers=int(need("num_hidden_layers")),
            num_attention_heads=n_q,
            num_key_value_heads=int(raw.get("num_key_value_heads") or n_q),
            head_dim=int(head_dim),
            intermediate_size=int(need("intermediate_size")),
            vocab_size=int(need("vocab_size")),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)),
            rope_theta=float(rope_theta),
            max_position_embeddings=int(raw.get("max_position_embeddings", 32768)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            attention_bias=bool(raw.get("attention_bias", False)),
            hidden_act=str(raw.get("hidden_act", "silu")),
            torch_dtype=str(raw.get("torch_dtype") or raw.get("dtype") or "bfloat16"),
            eos_token_ids=eos,
        )
        cfg.check()
        return cfg

    def check(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_dim % 2:
            raise ConfigError("head_dim must be even for rotary position encoding")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r}: this architecture uses silu")
        for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
                  "intermediate_size", "vocab_size", "max_position_embeddings"):
            if getattr(self, k) <= 0:
                raise ConfigError(f"{k} must be positive")

    def to_dict(self) -> Dict[str, Any]:
        """config.json content for a model folder of this configuration."""
        d = dataclasses.asdict(self)
        eos = d.pop("eos_token_ids")
        d["eos_token_id"] = eos[0] if len(eos) == 1 else (eos or None)
        d["architectures"] = ["Qwen3ForCausalLM"]
        d["model_type"] = "qwen3"
        return d


# what a Qwen3 checkpoint calls the parts of a layer (mini_sglang/models/qwen3.py:137-160)
QWEN3_LAYER_NAMES = {"input": "input_layernorm", "post_mixer": "post_attention_layernorm", "mixer": "self_attn",
                     "feed_forward": "mlp"}


def build_qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    """embed -> N x (norm, attention, norm, SwiGLU) -> norm -> head
    (mini_sglang/models/qwen3.py:129-232); every layer the same kind, run once in order."""
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    rope = PartSpec("rope_neox", {"head_dim": cfg.head_dim, "rotary_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                  "max_positions": cfg.max_position_embeddings})
    layers = []
    for l in range(cfg.num_hidden_layers):
        mixer = PartSpec("paged_attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "scale": cfg.head_dim ** -0.5, "qkv_bias": cfg.attention_bias, "qk_norm": True,
            "qk_norm_eps": cfg.rms_norm_eps, "window": None})
        ffn = PartSpec("swiglu_mlp", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
        layers.append(LayerSpec(prefix=f"model.layers.{l}", mixer=mixer, feed_forward=ffn,
                                norms={"input": norm, "post_mixer": norm}, position=rope, names=QWEN3_LAYER_NAMES))
    return ModelSpec(
        architecture="Qwen3ForCausalLM",
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                               "name": "model.embed_tokens.weight"}),
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps, "name": "model.norm.weight"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                  "tied": cfg.tie_word_embeddings, "name": "lm_head.weight",
                                  "tied_to": "model.embed_tokens.weight"}),
        layers=layers,
        schedule=[Run(layer=l, cache=l) for l in range(cfg.num_hidden_layers)],
        max_context_len=cfg.max_position_embeddings,
        eos_token_ids=list(cfg.eos_token_ids),
        checkpoint_dtype=cfg.torch_dtype,
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3_spec)
