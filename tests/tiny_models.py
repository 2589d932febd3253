"""Tiny Qwen3 configurations and seeded random weights for the tests.

Two configurations that differ in every size and option (layers, width, heads, groups,
head size, feed-forward width, vocabulary, rope base, eps, tied head), plus a third with an
odd group count.  Weights: matrices N(0, 0.02), norm weights 1 + N(0, 0.05), drawn in
float32 from a CPU generator seeded by (seed, tensor name) and rounded to bfloat16 so that
the bfloat16 engine, the float32 engine and the plain implementation all hold the same
numbers.  This file shares nothing with the engine package.
"""

from __future__ import annotations

import hashlib
import json
import os
import struct
from typing import Dict

import torch

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "intermediate_size": 128,
    "vocab_size": 256,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "max_position_embeddings": 512,
    "hidden_act": "silu",
    "attention_bias": False,
    "torch_dtype": "bfloat16",
    "eos_token_id": 255,
}

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 3,
    "hidden_size": 96,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 32,
    "intermediate_size": 160,
    "vocab_size": 320,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 1024,
    "hidden_act": "silu",
    "attention_bias": False,
    "torch_dtype": "bfloat16",
    "eos_token_id": 7,
}

# odd sizes: 3 kv heads, group of 5, head size 48, width and vocabulary no power of two
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 120,
    "num_attention_heads": 15,
    "num_key_value_heads": 3,
    "head_dim": 48,
    "intermediate_size": 200,
    "vocab_size": 333,
    "rope_theta": 50000.0,
    "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False,
    "max_position_embeddings": 2048,
    "hidden_act": "silu",
    "attention_bias": True,
    "torch_dtype": "bfloat16",
    "eos_token_id": 1,
}

CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C}


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    H = cfg["hidden_size"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or H // nq
    I, V = cfg["intermediate_size"], cfg["vocab_size"]
    out = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    if not cfg.get("tie_word_embeddings", False):
        out["lm_head.weight"] = (V, H)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        out[p + "input_layernorm.weight"] = (H,)
        out[p + "post_attention_layernorm.weight"] = (H,)
        out[p + "self_attn.q_proj.weight"] = (nq * d, H)
        out[p + "self_attn.k_proj.weight"] = (nkv * d, H)
        out[p + "self_attn.v_proj.weight"] = (nkv * d, H)
        out[p + "self_attn.o_proj.weight"] = (H, nq * d)
        out[p + "self_attn.q_norm.weight"] = (d,)
        out[p + "self_attn.k_norm.weight"] = (d,)
        if cfg.get("attention_bias", False):
            out[p + "self_attn.q_proj.bias"] = (nq * d,)
            out[p + "self_attn.k_proj.bias"] = (nkv * d,)
            out[p + "self_attn.v_proj.bias"] = (nkv * d,)
        out[p + "mlp.gate_proj.weight"] = (I, H)
        out[p + "mlp.up_proj.weight"] = (I, H)
        out[p + "mlp.down_proj.weight"] = (H, I)
    return out


def make_weights(cfg: dict, seed: int, std: float = 0.02) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors by checkpoint name."""
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
        g = torch.Generator(device="cpu").manual_seed(int.from_bytes(h[:7], "little"))
        if "norm" in name:
            t = 1.0 + 0.05 * torch.randn(shape, generator=g, dtype=torch.float32)
        else:
            t = std * torch.randn(shape, generator=g, dtype=torch.float32)
        out[name] = t.to(torch.bfloat16)
    return out


_ST_DTYPES = {torch.bfloat16: "BF16", torch.float32: "F32", torch.float16: "F16", torch.int32: "I32"}


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Minimal writer of the safetensors container (8-byte header length, JSON header, raw
    little-endian data), so that the tests do not depend on the engine's own writer."""
    header, blobs, off = {}, [], 0
    for name in sorted(tensors):
        t = tensors[name].contiguous().cpu()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _ST_DTYPES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def write_model_dir(path: str, cfg: dict, weights: Dict[str, torch.Tensor]) -> str:
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    write_safetensors(os.path.join(path, "model.safetensors"), weights)
    return path


def random_tokens(n: int, vocab: int, seed: int):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
