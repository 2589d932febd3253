"""One registry from the architecture's name (config.json `architectures[0]`) to its model.

(The reference builds Qwen3ForCausalLM unconditionally, mini_sglang/utils/loader.py:13-15, and reads the
configuration through transformers' AutoConfig, mini_sglang/utils/model_config.py.)

An architecture contributes two things: a typed configuration class that reads its own
config.json keys, and a function from that configuration to a ModelSpec.  Adding an
architecture is one `register_architecture` call; nothing else in the engine names it.
"""

from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Callable, Dict

from .spec import ModelSpec


@dataclasses.dataclass
class Architecture:
    name: str
    config_cls: Any                               # has .from_dict(dict) -> config
    build_spec: Callable[[Any], ModelSpec]        # config -> ModelSpec


ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: Any, build_spec: Callable[[Any], ModelSpec]) -> None:
    ARCHITECTURES[name] = Architecture(name, config_cls, build_spec)


class ConfigError(ValueError):
    pass


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    with open(path) as f:
        return json.load(f)


def architecture_of(raw: Dict[str, Any]) -> Architecture:
    names = raw.get("architectures") or []
    if not names:
        raise ConfigError("config.json has no `architectures` entry; known: " + ", ".join(sorted(ARCHITECTURES)))
    if names[0] not in ARCHITECTURES:
        raise ConfigError(f"unknown architecture {names[0]!r}; known: " + ", ".join(sorted(ARCHITECTURES)))
    return ARCHITECTURES[names[0]]


def load_config(model_dir: str):
    """-> (typed config, ModelSpec) for the model folder."""
    raw = read_config_json(model_dir)
    arch = architecture_of(raw)
    cfg = arch.config_cls.from_dict(raw)
    spec = arch.build_spec(cfg)
    spec.validate()
    return cfg, spec
