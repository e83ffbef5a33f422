"""Parts that only this file knows, registered and run without a change to the package: a feed-forward that
routes every token to one of several experts, and a position encoding that rotates a part of each head by a
scaled position.  They are toys that show what the parts' interfaces carry; they are no model of anyone's."""
import dataclasses
import math
from dataclasses import dataclass

import pytest
import torch

import plain_qwen3 as P
from helpers import CONFIG_B, CONFIG_C, cut, random_tokens, rel_err
from inferrs_b200 import kernels
from inferrs_b200.engine.batch import StepEntry
from inferrs_b200.engine.loading import spec_from_config
from inferrs_b200.engine.model import declared_tensors
from inferrs_b200.engine.runner import ModelRunner
from inferrs_b200.parts import TensorDecl
from inferrs_b200.parts.registry import register_feed_forward, register_position
from inferrs_b200.runtime import Runtime
from inferrs_b200.weights.random_init import random_weights

pytestmark = pytest.mark.gpu


def weights_for(decls, dtype, seed):
    w = random_weights(decls, seed, torch.bfloat16)            # values that bfloat16 holds exactly
    return {k: v.to(dtype).cuda() for k, v in w.items()}


def run_cut(runner, rid, toks, sizes):
    runner.admit(rid)
    rows, at = [], 0
    for n in cut(len(toks), sizes):
        rows.append(runner.step([StepEntry(rid, toks[at:at + n], list(range(n)))]))
        at += n
    runner.release(rid)
    return torch.cat(rows)


# ---- a feed-forward with routing ----------------------------------------------------------------------

@dataclass(frozen=True)
class ToyRoutedSpec:
    """Every token goes to the expert with the largest router logit (float32); the expert is a gated dense
    feed-forward of its own, and its output is weighted with the softmax probability of the choice."""
    width: int
    inner: int
    n_experts: int
    prefix: str
    kind: str = "toy_routed"


class ToyRouted:
    @staticmethod
    def declare(spec):
        out = [TensorDecl(f"{spec.prefix}.router.weight", (spec.n_experts, spec.width))]
        for e in range(spec.n_experts):
            out += [TensorDecl(f"{spec.prefix}.experts.{e}.gate_proj.weight", (spec.inner, spec.width)),
                    TensorDecl(f"{spec.prefix}.experts.{e}.up_proj.weight", (spec.inner, spec.width)),
                    TensorDecl(f"{spec.prefix}.experts.{e}.down_proj.weight", (spec.width, spec.inner))]
        return out

    def __init__(self, spec, weights, rt):
        self.spec, self.rt = spec, rt
        self.router = weights[f"{spec.prefix}.router.weight"].float()
        self.gate_up = [torch.cat([weights[f"{spec.prefix}.experts.{e}.gate_proj.weight"],
                                   weights[f"{spec.prefix}.experts.{e}.up_proj.weight"]]).contiguous()
                        for e in range(spec.n_experts)]
        self.down = [weights[f"{spec.prefix}.experts.{e}.down_proj.weight"].contiguous()
                     for e in range(spec.n_experts)]

    def forward(self, ctx, h):
        s = self.spec
        prob = torch.softmax(h.float() @ self.router.t(), dim=-1)      # the flat rows of the step, any cutting
        weight, choice = prob.max(dim=-1)
        y = torch.zeros((h.shape[0], s.width), dtype=self.rt.dtype, device=h.device)
        for e in range(s.n_experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            he = h[rows].contiguous()
            a = torch.empty((rows.numel(), s.inner), dtype=self.rt.dtype, device=h.device)
            kernels.gated_linear(he, self.gate_up[e], a, self.rt.dtype)
            ye = torch.empty((rows.numel(), s.width), dtype=self.rt.dtype, device=h.device)
            kernels.linear(a, self.down[e], ye, self.rt.dtype)
            y[rows] = (ye.float() * weight[rows, None]).to(self.rt.dtype)
        return y


def plain_routed(x, w, prefix, n_experts):
    prob = torch.softmax(x @ w[f"{prefix}.router.weight"].t(), dim=-1)
    weight, choice = prob.max(dim=-1)
    y = torch.zeros_like(x)
    for e in range(n_experts):
        rows = choice == e
        g = x[rows] @ w[f"{prefix}.experts.{e}.gate_proj.weight"].t()
        u = x[rows] @ w[f"{prefix}.experts.{e}.up_proj.weight"].t()
        y[rows] = ((P.silu(g) * u) @ w[f"{prefix}.experts.{e}.down_proj.weight"].t()) * weight[rows, None]
    return y, choice


def test_a_feed_forward_with_routing_is_registered_built_and_stepped():
    register_feed_forward("toy_routed", ToyRouted, replace=True)
    cfg = CONFIG_B
    spec, _ = spec_from_config(cfg)
    layers = list(spec.layers)
    toy = ToyRoutedSpec(width=cfg["hidden_size"], inner=40, n_experts=3, prefix="model.layers.1.toy_moe")
    layers[1] = layers[1].with_part("feed_forward", toy)
    spec = dataclasses.replace(spec, layers=tuple(layers))
    names = [d.name for d in declared_tensors(spec)]
    assert f"{toy.prefix}.router.weight" in names and "model.layers.1.mlp.gate_proj.weight" not in names
    rt = Runtime.cuda(torch.float32)
    weights = weights_for(declared_tensors(spec), torch.float32, seed=12)
    weights[f"{toy.prefix}.router.weight"] *= 50.0          # choices that no rounding changes
    runner = ModelRunner(spec, weights, rt, page_size=16, n_pages=16, max_requests=2)
    assert runner.graphs is None, "a part that does not declare graph_safe keeps the step out of CUDA graphs"
    toks = random_tokens(90, cfg["vocab_size"], seed=31)

    w = {k: v.float().cpu() for k, v in weights.items()}
    cos, sin = P.rope_tables(cfg["head_dim"], cfg["rope_theta"], len(toks), torch.float32)
    x = P.embedding(torch.tensor(toks), w["model.embed_tokens.weight"])
    used = None
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}"
        h = P.rms_norm(x, w[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
        x = x + P.attention_layer(h, w, f"{p}.self_attn", cfg, cos, sin)
        h = P.rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        if layer == 1:
            y, used = plain_routed(h, w, toy.prefix, toy.n_experts)
            x = x + y
        else:
            x = x + P.mlp(h, w, f"{p}.mlp")
    want = P.linear(P.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]), w["lm_head.weight"])
    assert len(set(used.tolist())) == 3, "the test wants every expert to get tokens"

    assert rel_err(run_cut(runner, "whole", toks, [90]).cpu(), want) < 1e-4
    assert rel_err(run_cut(runner, "cut", toks, [7, 2, 30, 1, 1, 13]).cpu(), want) < 1e-4


# ---- another position encoding ------------------------------------------------------------------------

@dataclass(frozen=True)
class ToyScaledRotarySpec:
    """The first ``rot_dim`` elements of every head are rotated by position / factor; the rest stay."""
    rot_dim: int
    theta: float
    max_positions: int
    factor: float
    kind: str = "toy_scaled_rotary"


class ToyScaledRotary:
    def __init__(self, spec, rt):
        half = spec.rot_dim // 2
        inv_freq = 1.0 / torch.pow(torch.tensor(float(spec.theta)), torch.arange(half, dtype=torch.float32) * 2.0 / spec.rot_dim)
        angle = (torch.arange(spec.max_positions, dtype=torch.float32) / spec.factor)[:, None] * inv_freq[None, :]
        self.cos, self.sin, self.rot_dim = torch.cos(angle).to(rt.device), torch.sin(angle).to(rt.device), spec.rot_dim

    def tables(self):
        return self.cos, self.sin, self.rot_dim


class ToyInterleavedRotary(ToyScaledRotary):
    """The same tables, but element 2i of a head turns with element 2i + 1 (the attribute is all it takes)."""
    interleaved = True


def plain_partial_rope(x, cos, sin, rot_dim, interleaved=False):
    if interleaved:
        x1, x2, rest = x[..., 0:rot_dim:2], x[..., 1:rot_dim:2], x[..., rot_dim:]
        turned = torch.stack([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).flatten(-2)
        return torch.cat([turned, rest], dim=-1)
    half = rot_dim // 2
    x1, x2, rest = x[..., :half], x[..., half:rot_dim], x[..., rot_dim:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos, rest], dim=-1)


@pytest.mark.parametrize("interleaved", [False, True], ids=["halves", "interleaved"])
@pytest.mark.parametrize("dtype,cfg", [(torch.float32, CONFIG_B), (torch.bfloat16, CONFIG_C)])
def test_another_position_encoding_is_registered_built_and_stepped(dtype, cfg, interleaved):
    register_position("toy_scaled_rotary", ToyScaledRotary, replace=True)
    register_position("toy_interleaved_rotary", ToyInterleavedRotary, replace=True)
    spec, _ = spec_from_config(cfg)
    d = cfg["head_dim"]
    toy = ToyScaledRotarySpec(rot_dim=d // 2, theta=500.0, max_positions=cfg["max_position_embeddings"], factor=4.0,
                              kind="toy_interleaved_rotary" if interleaved else "toy_scaled_rotary")
    layers = tuple(l.with_part("mixer", dataclasses.replace(l.mixer, position=toy)) for l in spec.layers)
    spec = dataclasses.replace(spec, layers=layers)
    rt = Runtime.cuda(dtype)
    weights = weights_for(declared_tensors(spec), dtype, seed=14)
    runner = ModelRunner(spec, weights, rt, page_size=16, n_pages=16, max_requests=2)
    toks = random_tokens(100, cfg["vocab_size"], seed=33)

    store = None if dtype == torch.float32 else dtype
    rnd = (lambda t: t) if store is None else (lambda t: t.to(store).float())
    w = {k: v.float().cpu() for k, v in weights.items()}
    t, nh, nkv, eps = len(toks), cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["rms_norm_eps"]
    half = toy.rot_dim // 2
    inv_freq = 1.0 / torch.pow(torch.tensor(toy.theta), torch.arange(half, dtype=torch.float32) * 2.0 / toy.rot_dim)
    angle = (torch.arange(t, dtype=torch.float32) / toy.factor)[:, None] * inv_freq[None, :]
    cos, sin = torch.cos(angle), torch.sin(angle)
    x = P.embedding(torch.tensor(toks), w["model.embed_tokens.weight"])
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}"
        h = rnd(P.rms_norm(x, w[f"{p}.input_layernorm.weight"], eps))
        q = rnd(P.linear(h, w[f"{p}.self_attn.q_proj.weight"])).reshape(t, nh, d).transpose(0, 1)
        k = rnd(P.linear(h, w[f"{p}.self_attn.k_proj.weight"])).reshape(t, nkv, d).transpose(0, 1)
        v = rnd(P.linear(h, w[f"{p}.self_attn.v_proj.weight"])).reshape(t, nkv, d).transpose(0, 1)
        q = rnd(plain_partial_rope(P.rms_norm(q, w[f"{p}.self_attn.q_norm.weight"], eps), cos, sin, toy.rot_dim, interleaved))
        k = rnd(plain_partial_rope(P.rms_norm(k, w[f"{p}.self_attn.k_norm.weight"], eps), cos, sin, toy.rot_dim, interleaved))
        o = rnd(P.causal_attention(q, k, v, 1.0 / math.sqrt(d)))
        x = x + rnd(P.linear(o, w[f"{p}.self_attn.o_proj.weight"]))
        h = rnd(P.rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps))
        x = x + P.mlp(h, w, f"{p}.mlp", store)
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    want = P.linear(rnd(P.rms_norm(x, w["model.norm.weight"], eps)), head)

    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert rel_err(run_cut(runner, "whole", toks, [100]).cpu(), want) < tol
    assert rel_err(run_cut(runner, "cut", toks, [68] + [1] * 32).cpu(), want) < tol
    assert rel_err(run_cut(runner, "portions", toks, [5, 2, 40, 3]).cpu(), want) < tol
