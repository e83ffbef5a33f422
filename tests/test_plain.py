"""The plain implementation checked against itself and against hand-made cases."""
import math

import torch

import plain_qwen3 as P
from helpers import CONFIG_B, random_tokens


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    out = P.rms_norm(x, torch.tensor([2.0, 0.5]), 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[6.0 / r, 2.0 / r]]))


def test_rope_rotates_pairs_split_in_halves():
    cos, sin = P.rope_tables(4, 10000.0, 3, torch.float32)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]] * 3])   # one head, three positions
    y = P.rope(x, cos, sin)
    assert torch.allclose(y[0, 0], x[0, 0])            # position 0: no rotation
    a0, a1 = 1.0, 1.0 / 100.0                          # angles at position 1: theta^(-0/4), theta^(-2/4)
    want = torch.tensor([1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                         1 * math.sin(a0) + 3 * math.cos(a0), 2 * math.sin(a1) + 4 * math.cos(a1)])
    assert torch.allclose(y[0, 1], want, atol=1e-6)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(4, 6, 8), torch.randn(2, 6, 8), torch.randn(2, 6, 8)
    o = P.causal_attention(q, k, v, 0.3)
    o_short = P.causal_attention(q[:, :4], k[:, :4], v[:, :4], 0.3)
    assert torch.allclose(o[:4], o_short, atol=1e-6)              # later tokens change nothing earlier
    assert torch.allclose(o[0, :16].reshape(2, 8), v[0, 0].expand(2, 8))   # heads 0,1 read kv head 0
    assert torch.allclose(o[0, 16:].reshape(2, 8), v[1, 0].expand(2, 8))   # heads 2,3 read kv head 1
    w = P.causal_attention(q, k, v, 0.3, window=1)
    assert torch.allclose(w.reshape(6, 2, 2, 8)[:, :, 0], v.transpose(0, 1), atol=1e-6)  # only itself


def test_silu():
    z = torch.tensor([0.0, 1.0, -2.0])
    assert torch.allclose(P.silu(z), z * torch.sigmoid(z))


def test_float64_agrees_and_prefix_property(model_dirs):
    cfg, w = P.read_model(model_dirs["B"])
    toks = random_tokens(50, CONFIG_B["vocab_size"], seed=9)
    l32 = P.forward(cfg, w, toks)
    l64 = P.forward(cfg, w, toks, dtype=torch.float64)
    assert float((l32.double() - l64).abs().max() / l64.abs().max()) < 2e-5
    assert torch.allclose(P.forward(cfg, w, toks[:20]), l32[:20], atol=1e-5)
    assert l32.shape == (50, CONFIG_B["vocab_size"])
    lb = P.forward(cfg, w, toks, store=torch.bfloat16)
    assert 1e-4 < float((lb - l32).abs().max() / l32.abs().max()) < 5e-2   # rounding is there, and small
