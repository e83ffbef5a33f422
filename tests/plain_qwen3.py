"""A plain, slow Qwen3 decoder: whole sequences, no cache, one function per part.

It rests on the reference's formulas, not on its compiled code: the reference
is a Rust workspace and there is no Rust toolchain on the machines this was
written on, so its model code can be neither imported nor compiled here.  Each
function cites the lines of the reference that give its formula.

It shares no code with the package: it reads config.json with ``json`` and the
weights with the ``safetensors`` library, and it knows nothing of pages, steps
or batches.  ``forward`` returns the logits of every position of one sequence.

``store`` names the dtype in which the product keeps activations between its
kernels (``None``: nothing is rounded).  With ``store=torch.bfloat16`` values
are rounded to bfloat16 at the places where the product stores them in
bfloat16; sums, norms, softmax and rotation stay in ``dtype`` as they do there.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


def read_model(model_dir: str, dtype=torch.float32):
    """config.json as a dict and every tensor as ``dtype``."""
    from safetensors import safe_open

    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    weights = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return config, weights


def _rnd(x: torch.Tensor, store) -> torch.Tensor:
    return x if store is None else x.to(store).to(x.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Row gather, no scale (inferrs-models/src/models/qwen3.rs:399, candle-nn/src/embedding.rs:27-36)."""
    return table[ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last dimension
    (candle-nn/src/ops.rs:480-494; inferrs-kernels/candle-kernels/src/reduce.cu:188-228)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * weight


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y = x W^T with W stored [out, in], no bias (candle-nn/src/linear.rs:41-82, qwen3.rs:76-79)."""
    return x @ weight.t()


def rope_tables(head_dim: int, theta: float, n_positions: int, dtype) -> (torch.Tensor, torch.Tensor):
    """inv_freq_i = 1 / theta^(2i/d) and angle = position * inv_freq_i, both in 32-bit
    (inferrs-models/src/models/attention_utils.rs:186-216)."""
    half = head_dim // 2
    exponent = torch.arange(half, dtype=torch.float32) * 2.0 / float(head_dim)
    inv_freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), exponent)
    pos = torch.arange(n_positions, dtype=torch.float32)
    angle = pos[:, None] * inv_freq[None, :]
    return torch.cos(angle).to(dtype), torch.sin(angle).to(dtype)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Split-half rotation of x [heads, t, d]: o_i = x_i c - x_{i+d/2} s, o_{i+d/2} = x_i s + x_{i+d/2} c
    (attention_utils.rs:137-151; reduce.cu:292-312)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int] = None) -> torch.Tensor:
    """q [nh, t, d], k/v [nkv, t, d] -> [t, nh*d].

    Query head h reads key/value head h // (nh/nkv) (attention_utils.rs:38-49);
    scores = q k^T * scale (qwen3.rs:165-175); key j is visible to query i iff
    j <= i (attention_utils.rs:61-85); softmax over keys (reduce.cu:232-272);
    output = P v, heads side by side (qwen3.rs:186-192).  ``window`` is not part
    of the reference's Qwen3; it restricts keys to i - window < j <= i for the
    tests of the cache's window groups.
    """
    nh, t, d = q.shape
    nkv = k.shape[0]
    g = nh // nkv
    k = k.repeat_interleave(g, dim=0)
    v = v.repeat_interleave(g, dim=0)
    s = (q @ k.transpose(1, 2)) * scale
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & (j > i - window)
    s = s.masked_fill(~visible, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = p @ v
    return o.transpose(0, 1).reshape(t, nh * d)


def attention_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict, cos, sin,
                    store=None, window=None) -> torch.Tensor:
    """Projections, per-head q/k norm, rotation, attention, output projection (qwen3.rs:104-196)."""
    t = x.shape[0]
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = _rnd(linear(x, w[f"{prefix}.q_proj.weight"]), store).reshape(t, nh, d).transpose(0, 1)
    k = _rnd(linear(x, w[f"{prefix}.k_proj.weight"]), store).reshape(t, nkv, d).transpose(0, 1)
    v = _rnd(linear(x, w[f"{prefix}.v_proj.weight"]), store).reshape(t, nkv, d).transpose(0, 1)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], eps)   # qwen3.rs:128-129: before the rotation
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], eps)
    q = _rnd(rope(q, cos[:t], sin[:t]), store)
    k = _rnd(rope(k, cos[:t], sin[:t]), store)
    o = _rnd(causal_attention(q, k, v, 1.0 / math.sqrt(d), window), store)
    return _rnd(linear(o, w[f"{prefix}.o_proj.weight"]), store)


def silu(z: torch.Tensor) -> torch.Tensor:
    """z / (1 + exp(-z)) (inferrs-kernels/candle-kernels/src/unary.cu:58-61)."""
    return z / (1.0 + torch.exp(-z))


def mlp(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, store=None) -> torch.Tensor:
    """down( silu(gate(x)) * up(x) ) (attention_utils.rs:94-118)."""
    g = _rnd(linear(x, w[f"{prefix}.gate_proj.weight"]), store)
    u = _rnd(linear(x, w[f"{prefix}.up_proj.weight"]), store)
    a = _rnd(silu(g) * u, store)
    return _rnd(linear(a, w[f"{prefix}.down_proj.weight"]), store)


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], layer: int, cfg: dict, cos, sin,
                  store=None, window=None) -> torch.Tensor:
    """x += attention(norm(x)); x += mlp(norm(x)) (qwen3.rs:285-300)."""
    p = f"model.layers.{layer}"
    eps = cfg["rms_norm_eps"]
    h = _rnd(rms_norm(x, w[f"{p}.input_layernorm.weight"], eps), store)
    x = x + attention_layer(h, w, f"{p}.self_attn", cfg, cos, sin, store, window)
    h = _rnd(rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps), store)
    return x + mlp(h, w, f"{p}.mlp", store)


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: List[int], dtype=torch.float32, store=None,
            windows: Optional[List[Optional[int]]] = None, last: Optional[int] = None) -> torch.Tensor:
    """Logits [t, vocab] of every position of one sequence (qwen3.rs:398-407; the reference keeps
    only the last row, attention_utils.rs:382-395).  ``last``: only the logits of that many last positions."""
    cfg = dict(cfg)
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    w = {k: v.to(dtype) for k, v in w.items()}
    ids_t = torch.tensor(ids, dtype=torch.long)
    cos, sin = rope_tables(cfg["head_dim"], cfg["rope_theta"], len(ids), dtype)
    x = embedding(ids_t, w["model.embed_tokens.weight"])
    for layer in range(cfg["num_hidden_layers"]):
        win = windows[layer] if windows is not None else None
        x = decoder_layer(x, w, layer, cfg, cos, sin, store, win)
    if last is not None:
        x = x[-last:]
    x = _rnd(rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]), store)
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]  # qwen3.rs:366-373
    return linear(x, head)
