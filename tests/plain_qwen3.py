"""Plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache.

Written from the formulas of jason-fxz/mini-sglang (paths below are relative to that
project).  One function per part; float32 or float64 torch arithmetic on whatever device
the inputs live on; nothing is shared with the engine's product path (no import from
the engine package).  tests/golden/make_golden.py checks this file once against the
reference project's own model code on the CPU; the small outputs of that run are
committed under tests/golden/.

Weights are a dict {checkpoint tensor name: tensor}; the configuration is the dict
read from config.json.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h = E[ids]; no scaling (mini_sglang/layers/embed_head.py:49, models/qwen3.py:202)."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, plain weight (mini_sglang/layers/layernorm.py:39-46)."""
    var = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float, dtype) -> tuple:
    """inv_freq_i = theta^(-2i/d); angle[p, i] = p * inv_freq_i
    (mini_sglang/layers/rotary_embedding.py:59-66).  The reference builds the table in
    float32; `dtype` lets the oracle use float64 as well."""
    idx = torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device)
    inv_freq = 1.0 / (theta ** (idx / head_dim))
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    return ang.cos().to(dtype), ang.sin().to(dtype)


def rope_neox(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, d]; halves rotated against each other
    (mini_sglang/layers/rotary_embedding.py:19-33)."""
    x1, x2 = torch.chunk(x, 2, dim=-1)
    c = cos[:, None, :]
    s = sin[:, None, :]
    return torch.cat((x1 * c - x2 * s, x1 * s + x2 * c), dim=-1)


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                         window: Optional[int] = None) -> torch.Tensor:
    """q: [S, n_q, d], k/v: [S, n_kv, d] of ONE whole sequence.  Query head h reads kv head
    h // (n_q / n_kv); keys after the query are masked; softmax over the rest; scale d^-0.5
    (mini_sglang/models/qwen3.py:50, layers/attn/torch_attn_backend.py:63-111).
    `window` (not used by Qwen3 in the reference) keeps only the last `window` keys."""
    S, n_q, d = q.shape
    n_kv = k.shape[1]
    g = n_q // n_kv
    out = torch.empty_like(q)
    pos = torch.arange(S, device=q.device)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > (pos[:, None] - window)
    for h in range(n_q):
        kh = k[:, h // g, :]
        vh = v[:, h // g, :]
        s = (q[:, h, :] @ kh.T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ vh
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up (mini_sglang/layers/activation.py:12-14)."""
    return torch.nn.functional.silu(gate) * up


def attention_block(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict,
                    positions: torch.Tensor) -> torch.Tensor:
    """qkv projection, per-head q_norm/k_norm before RoPE, attention, o_proj
    (mini_sglang/models/qwen3.py:86-97)."""
    n_q = cfg["num_attention_heads"]
    n_kv = cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // n_q
    eps = cfg["rms_norm_eps"]
    S = x.shape[0]
    q = x @ w[prefix + "q_proj.weight"].T
    k = x @ w[prefix + "k_proj.weight"].T
    v = x @ w[prefix + "v_proj.weight"].T
    if cfg.get("attention_bias", False):
        q = q + w[prefix + "q_proj.bias"]
        k = k + w[prefix + "k_proj.bias"]
        v = v + w[prefix + "v_proj.bias"]
    q = rms_norm(q.reshape(S, n_q, d), w[prefix + "q_norm.weight"], eps)
    k = rms_norm(k.reshape(S, n_kv, d), w[prefix + "k_norm.weight"], eps)
    v = v.reshape(S, n_kv, d)
    cos, sin = rope_angles(positions, d, float(cfg.get("rope_theta", 1000000.0)), x.dtype)
    q = rope_neox(q, cos, sin)
    k = rope_neox(k, cos, sin)
    o = causal_gqa_attention(q, k, v, d ** -0.5)
    return o.reshape(S, n_q * d) @ w[prefix + "o_proj.weight"].T


def mlp_block(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) (mini_sglang/models/qwen3.py:122-126)."""
    g = x @ w[prefix + "gate_proj.weight"].T
    u = x @ w[prefix + "up_proj.weight"].T
    return swiglu(g, u) @ w[prefix + "down_proj.weight"].T


def forward_sequence(cfg: dict, weights: Dict[str, torch.Tensor], token_ids: List[int],
                     dtype=torch.float32, device="cpu", rows: Optional[List[int]] = None) -> torch.Tensor:
    """Logits [S, vocab] at every position of one whole sequence (or, with `rows`, at those positions only:
    the whole sequence is computed all the same, only the head is spared for the others).

    Residual convention of mini_sglang/models/qwen3.py:169-178,203-206: the stream `res`
    collects x + attn + mlp; every norm reads the updated stream."""
    w = {k: v.to(device=device, dtype=dtype) for k, v in weights.items()}
    ids = torch.tensor(token_ids, dtype=torch.long, device=device)
    positions = torch.arange(len(token_ids), device=device)
    eps = cfg["rms_norm_eps"]
    res = embed(ids, w["model.embed_tokens.weight"])
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        y = rms_norm(res, w[p + "input_layernorm.weight"], eps)
        res = res + attention_block(y, w, p + "self_attn.", cfg, positions)
        y = rms_norm(res, w[p + "post_attention_layernorm.weight"], eps)
        res = res + mlp_block(y, w, p + "mlp.")
    if rows is not None:
        res = res[torch.tensor(rows, dtype=torch.long, device=device)]
    h = rms_norm(res, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return h @ head.T      # mini_sglang/layers/logits_processor.py:56-59


def greedy_generate(cfg: dict, weights: Dict[str, torch.Tensor], prompt: List[int], n_new: int,
                    dtype=torch.float32, device="cpu") -> List[int]:
    """Greedy continuation by re-running the whole sequence for every new token
    (argmax: mini_sglang/layers/sampler.py:15)."""
    toks = list(prompt)
    for _ in range(n_new):
        logits = forward_sequence(cfg, weights, toks, dtype=dtype, device=device)
        toks.append(int(logits[-1].argmax().item()))
    return toks[len(prompt):]


# ---------------------------------------------------------------------------------------
# sampling (mini_sglang/layers/sampler.py:13-23), with the noise given from outside
# ---------------------------------------------------------------------------------------

def sample_with_noise(logits: torch.Tensor, temperatures: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
    """greedy where T == 0, else argmax(softmax(logits / T) / (noise + 1e-10)) with
    noise ~ Exp(1) drawn by the caller."""
    logits = logits.to(torch.float32)
    greedy = logits.argmax(dim=-1)
    t = torch.where(temperatures == 0, torch.ones_like(temperatures), temperatures)
    probs = torch.softmax(logits / t[:, None], dim=-1, dtype=torch.float32)
    sampled = (probs / (noise + 1e-10)).argmax(dim=-1)
    return torch.where(temperatures == 0, greedy, sampled)


# Philox4x32-10 in plain integers: the counter-based generator the engine's sampling
# kernel is specified to use (key = seed lo/hi, counter = (vocab index // 4, row key, 0, 0)).
_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def philox4x32(counter, key):
    c = list(counter)
    k = list(key)
    for _ in range(10):
        p0 = _M0 * c[0]
        p1 = _M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & _MASK, p1 & _MASK,
             ((p0 >> 32) ^ c[3] ^ k[1]) & _MASK, p0 & _MASK]
        k = [(k[0] + _W0) & _MASK, (k[1] + _W1) & _MASK]
    return c


def exponential_noise(seed: int, row_key: int, step: int, vocab: int) -> torch.Tensor:
    """Exp(1) noise for one row: word j % 4 of Philox(counter=(j // 4, row_key, step, 0), key=seed)
    -> u = ((word >> 9) + 0.5) * 2^-23, exact in float32 and strictly inside (0, 1) -> -log(u)."""
    key = (seed & _MASK, (seed >> 32) & _MASK)
    us = []
    for blk in range((vocab + 3) // 4):
        words = philox4x32((blk, row_key & _MASK, step & _MASK, 0), key)
        us.extend(((wd >> 9) + 0.5) * (2.0 ** -23) for wd in words)
    u = torch.tensor(us[:vocab], dtype=torch.float32)
    return -torch.log(u)
