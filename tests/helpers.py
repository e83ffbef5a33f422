"""Tiny configurations and the ways of cutting a request into steps that the tests share."""
from __future__ import annotations

import random
from typing import Dict, List, Sequence

import torch

# Two configurations of the architecture that differ in every size and option.
CONFIG_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 512, "tie_word_embeddings": True, "hidden_act": "silu",
}
CONFIG_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 8, "num_key_value_heads": 2,
    "head_dim": 32, "intermediate_size": 272, "vocab_size": 517, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "max_position_embeddings": 640, "tie_word_embeddings": False, "hidden_act": "silu",
}
# A third shape whose head size the tensor-core attention kernels take (A and B run the generic kernel).
CONFIG_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 160, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 208, "vocab_size": 301, "rope_theta": 50000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 768, "tie_word_embeddings": True, "hidden_act": "silu",
}
# A fourth shape with the head size of the published checkpoints (128): the bfloat16 engine then runs the TMA and
# tcgen05 attention kernels and, in decode steps, the tcgen05 matrix product under programmatic dependent launch.
CONFIG_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 328, "vocab_size": 389, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 1024, "tie_word_embeddings": False, "hidden_act": "silu",
}
PAGE_SIZE = {"A": 4, "B": 16, "C": 16, "D": 16}


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def cut(n: int, sizes: Sequence[int]) -> List[int]:
    """Cut n tokens into portions, cycling through ``sizes``; the last portion takes what is left."""
    out, i = [], 0
    while n > 0:
        s = min(sizes[i % len(sizes)], n)
        out.append(s)
        n -= s
        i += 1
    return out


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """The worst row's error: for every row (last dimension) the largest absolute difference over the largest
    absolute value of the reference ``b`` in that row; the largest of these.  One bad row among hundreds, or an
    error in a row of small values, shows in full."""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    if a.shape != b.shape:
        raise ValueError(f"shapes differ: {tuple(a.shape)} and {tuple(b.shape)}")
    if a.dim() == 0:
        a, b = a.reshape(1, 1), b.reshape(1, 1)
    elif a.dim() == 1:
        a, b = a.reshape(1, -1), b.reshape(1, -1)
    a, b = a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1])
    if a.numel() == 0:
        return 0.0
    if not bool(torch.isfinite(a).all()):
        return float("inf")
    diff = (a - b).abs().amax(dim=1)
    scale = b.abs().amax(dim=1).clamp_min(1e-30)
    return float((diff / scale).max())
