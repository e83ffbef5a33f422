"""A norm and a block arrangement that only this file knows, registered from here and run through the engine without a
change to the package.

The norm subtracts the mean, divides by the standard deviation and has a weight and a bias; it gives no sink, so no
product ever folds it in.  The arrangement lets both sub-layers of a layer read the same normalised rows and adds both
outputs to the residual stream at once ("parallel" sub-layers).  The toy model has a parallel layer of the package's own
attention and gated feed-forward, then an ordinary sequential layer whose norms are the toy norm (so the sequential
block meets norms without a sink), then a sequential layer with the package's own norms (whose products may fold them).
It is no model of anyone's; every part of it says ``graph_safe``, so its steps are replayed graphs.
"""
import math
from dataclasses import dataclass

import pytest
import torch

import plain_qwen3 as P
from helpers import random_tokens, rel_err
from inferrs_b200 import Engine, SamplingParams
from inferrs_b200.config.base import ConfigError, RawConfig, register_architecture
from inferrs_b200.engine.batch import StepEntry
from inferrs_b200.parts import (AttentionSpec, GatedDenseSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec,
                                ScheduleEntry, SubLayerSpec, TensorDecl, pre_norm_layer, register_arrangement,
                                register_norm)

pytestmark = pytest.mark.gpu

CONFIGS = {
    "a": {"architectures": ["ToyParallelLM"], "width": 88, "inner": 136, "vocab": 307, "heads": 6, "kv_heads": 2,
          "head_dim": 16, "theta": 7000.0, "eps": 1e-5, "positions": 384},
    "b": {"architectures": ["ToyParallelLM"], "width": 48, "inner": 200, "vocab": 97, "heads": 3, "kv_heads": 3,
          "head_dim": 32, "theta": 30000.0, "eps": 3e-6, "positions": 192},
}


@dataclass(frozen=True)
class ToyConfig:
    width: int
    inner: int
    vocab: int
    heads: int
    kv_heads: int
    head_dim: int
    theta: float
    eps: float
    positions: int

    @classmethod
    def from_raw(cls, raw: RawConfig) -> "ToyConfig":
        ints = ("width", "inner", "vocab", "heads", "kv_heads", "head_dim", "positions")
        floats = ("theta", "eps")
        missing = [k for k in ints + floats if not raw.has(k)]
        if missing:
            raise ConfigError(f"{raw.source}: the toy config lacks {missing}")
        return cls(**{k: raw.get_int(k) for k in ints}, **{k: raw.get_float(k) for k in floats})


@dataclass(frozen=True)
class ToyCenterNormSpec:
    size: int
    eps: float
    weight: str
    bias: str
    kind: str = "toy_center"


class ToyCenterNorm:
    """(x - mean) / sqrt(var + eps) * w + b over the width, in float32."""

    graph_safe = True

    @staticmethod
    def declare(spec):
        return [TensorDecl(spec.weight, (spec.size,), init="norm"), TensorDecl(spec.bias, (spec.size,))]

    def __init__(self, spec, weights, rt):
        self.spec, self.rt = spec, rt
        self.weight, self.bias = weights[spec.weight].float(), weights[spec.bias].float()

    def _center(self, x: torch.Tensor) -> torch.Tensor:
        x = x - x.mean(-1, keepdim=True)
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.spec.eps) * self.weight + self.bias

    def add_norm(self, residual, delta, rows=None):
        if rows is not None:                                  # a choice of rows: nothing is written back
            x = residual.index_select(0, rows.long())
            if delta is not None:
                x = x + delta.index_select(0, rows.long()).float()
            return self._center(x).to(self.rt.dtype)
        if delta is not None:
            residual.add_(delta.float())
        return self._center(residual).to(self.rt.dtype)

    def norm(self, x):
        return self._center(x.float()).to(x.dtype)


class ToyParallelBlock:
    """x += sum over the sub-layers of part(norm(x)), all of them reading the same rows: the first sub-layer's norm is
    the layer's norm.  What the block before handed on is added first; this block's own sum is handed on."""

    def __init__(self, spec, sublayers):
        if not sublayers or any(s.post_norm is not None for s in sublayers):
            raise ValueError("a parallel block has sub-layers without norms after them")
        self.spec, self.sublayers = spec, list(sublayers)

    def parts(self):
        yield self.sublayers[0].norm
        for s in self.sublayers:
            yield s.part

    def forward(self, ctx, cache_id, residual, pending):
        h = self.sublayers[0].norm.add_norm(residual, pending)
        total = None
        for s in self.sublayers:
            y = s.run(ctx, cache_id, h)
            total = y if total is None else total + y
        return total


def build_spec(cfg: ToyConfig) -> ModelSpec:
    def rms(name):
        return NormSpec(size=cfg.width, eps=cfg.eps, weight=name)

    def center(prefix):
        return ToyCenterNormSpec(size=cfg.width, eps=cfg.eps, weight=f"{prefix}.weight", bias=f"{prefix}.bias")

    def dense(p):
        return GatedDenseSpec(width=cfg.width, inner=cfg.inner, gate_proj=f"{p}.gate_proj.weight",
                              up_proj=f"{p}.up_proj.weight", down_proj=f"{p}.down_proj.weight")

    position = PositionSpec(kind="rotary_split_half", rot_dim=cfg.head_dim, theta=cfg.theta, max_positions=cfg.positions)

    def attention(a):
        return AttentionSpec(
            width=cfg.width, n_heads=cfg.heads, n_kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
            scale=1.0 / math.sqrt(cfg.head_dim), position=position, q_proj=f"{a}.q_proj.weight",
            k_proj=f"{a}.k_proj.weight", v_proj=f"{a}.v_proj.weight", o_proj=f"{a}.o_proj.weight",
            q_norm=NormSpec(size=cfg.head_dim, eps=cfg.eps, weight=f"{a}.q_norm.weight"),
            k_norm=NormSpec(size=cfg.head_dim, eps=cfg.eps, weight=f"{a}.k_norm.weight"))

    layers = (
        LayerSpec(arrangement="toy_parallel", sublayers=(
            SubLayerSpec(part=attention("blocks.0.attn"), category="mixer", norm=center("blocks.0.norm")),
            SubLayerSpec(part=dense("blocks.0.mlp"), category="feed_forward"))),
        pre_norm_layer(center("blocks.1.n1"), attention("blocks.1.attn"), center("blocks.1.n2"), dense("blocks.1.mlp")),
        pre_norm_layer(rms("blocks.2.n1.weight"), attention("blocks.2.attn"), rms("blocks.2.n2.weight"),
                       dense("blocks.2.mlp")),
    )
    return ModelSpec(
        vocab_size=cfg.vocab, width=cfg.width, embedding="emb.weight", layers=layers,
        schedule=tuple(ScheduleEntry(layer=i, cache=i) for i in range(len(layers))),
        final_norm=center("final"), lm_head="head.weight", lm_head_optional=False, max_positions=cfg.positions,
        architecture="ToyParallelLM")


def register_toy():
    register_norm("toy_center", ToyCenterNorm, replace=True)
    register_arrangement("toy_parallel", ToyParallelBlock, replace=True)
    register_architecture("ToyParallelLM", ToyConfig, build_spec, replace=True)


def toy_engine(cfg: dict, dtype: str, **kw) -> Engine:
    register_toy()
    eng = Engine(config=cfg, random_weights=23, dtype=dtype, block_size=16, **kw)
    for blk in eng.runner.model.blocks:                       # biases that matter (they are drawn small)
        for p in blk.parts():
            if isinstance(p, ToyCenterNorm):
                p.bias.mul_(20.0)
    return eng


def host_weights(eng: Engine, cfg: dict) -> dict:
    m = eng.runner.model
    w = {"emb.weight": m.embedding, "head.weight": m.head.weight,
         "final.weight": m.final_norm.weight, "final.bias": m.final_norm.bias}
    nh, nkv, d = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    for b, blk in enumerate(m.blocks):
        a, f = blk.sublayers[0].part, blk.sublayers[1].part
        q, k, v = a.qkv.weight.split([nh * d, nkv * d, nkv * d])
        g, u = f.gate_up.weight.split([cfg["inner"], cfg["inner"]])
        p = f"blocks.{b}"
        w.update({f"{p}.attn.q_proj.weight": q, f"{p}.attn.k_proj.weight": k, f"{p}.attn.v_proj.weight": v,
                  f"{p}.attn.o_proj.weight": a.o.weight, f"{p}.attn.q_norm.weight": a.q_weight,
                  f"{p}.attn.k_norm.weight": a.k_weight, f"{p}.mlp.gate_proj.weight": g, f"{p}.mlp.up_proj.weight": u,
                  f"{p}.mlp.down_proj.weight": f.down.weight})
    n0 = m.blocks[0].sublayers[0].norm
    w.update({"blocks.0.norm.weight": n0.weight, "blocks.0.norm.bias": n0.bias})
    for s, name in zip(m.blocks[1].sublayers, ("n1", "n2")):
        w.update({f"blocks.1.{name}.weight": s.norm.weight, f"blocks.1.{name}.bias": s.norm.bias})
    for s, name in zip(m.blocks[2].sublayers, ("n1", "n2")):
        w[f"blocks.2.{name}.weight"] = s.norm.weight
    return {k: t.float().cpu() for k, t in w.items()}


def plain_forward(c: dict, w: dict, ids, store=None) -> torch.Tensor:
    """The toy as whole-sequence arithmetic (float32; ``store``: what a sub-layer hands on is rounded to it)."""
    def r(x):
        return x if store is None else x.to(store).float()

    def center(x, p):
        x = x - x.mean(-1, keepdim=True)
        return r(x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + c["eps"]) * w[f"{p}.weight"] + w[f"{p}.bias"])

    t = len(ids)
    acfg = {"num_attention_heads": c["heads"], "num_key_value_heads": c["kv_heads"], "head_dim": c["head_dim"],
            "rms_norm_eps": c["eps"]}
    cos, sin = P.rope_tables(c["head_dim"], c["theta"], t, torch.float32)
    x = P.embedding(torch.tensor(ids), w["emb.weight"])
    h = center(x, "blocks.0.norm")
    x = x + r(r(P.attention_layer(h, w, "blocks.0.attn", acfg, cos, sin, store=store)) +
              r(P.mlp(h, w, "blocks.0.mlp", store=store)))
    x = x + r(P.attention_layer(center(x, "blocks.1.n1"), w, "blocks.1.attn", acfg, cos, sin, store=store))
    x = x + r(P.mlp(center(x, "blocks.1.n2"), w, "blocks.1.mlp", store=store))
    x = x + r(P.attention_layer(r(P.rms_norm(x, w["blocks.2.n1.weight"], c["eps"])), w, "blocks.2.attn", acfg, cos, sin,
                                store=store))
    x = x + r(P.mlp(r(P.rms_norm(x, w["blocks.2.n2.weight"], c["eps"])), w, "blocks.2.mlp", store=store))
    return P.linear(center(x, "final"), w["head.weight"])


@pytest.mark.parametrize("name,dtype,tol", [("a", "f32", 1e-4), ("b", "f32", 1e-4), ("a", "bf16", 4e-2)])
def test_a_norm_and_an_arrangement_from_outside_are_registered_built_and_stepped(name, dtype, tol):
    cfg = CONFIGS[name]
    eng = toy_engine(cfg, dtype, num_blocks=40, max_batch_size=3, max_tokens_per_step=96)
    runner = eng.runner
    assert runner.graphs is not None, "every part of the toy says graph_safe: its steps are replayed graphs"
    w = host_weights(eng, cfg)
    toks = random_tokens(90, cfg["vocab"], seed=8)
    want = plain_forward(cfg, w, toks, store=None if dtype == "f32" else torch.bfloat16)
    runner.admit("whole")
    got = runner.step([StepEntry("whole", toks, list(range(len(toks))))])
    assert rel_err(got, want) < tol
    runner.release("whole")
    # in portions of changing size beside another request, the last tokens one by one (the steps of single tokens are
    # where the sequential layer with the package's own norms folds them into its products)
    other = random_tokens(50, cfg["vocab"], seed=9)
    runner.admit("cut")
    runner.admit("other")
    at, rows, o_at = 0, [], 0
    for n in (9, 2, 31, 17, 3, 12) + (1,) * 16:
        entries = [StepEntry("cut", toks[at:at + n], list(range(n)))]
        if o_at < len(other):
            m = 7 if n > 1 else 1
            entries.append(StepEntry("other", other[o_at:o_at + m], []))
            o_at += m
        rows.append(runner.step(entries)[:n])
        at += n
    assert at == len(toks)
    assert rel_err(torch.cat(rows), want) < tol
    runner.release("cut")
    runner.release("other")
    runner.manager.check_invariants()


def test_the_toy_generates_through_the_entry_point_what_its_plain_statement_says():
    cfg = CONFIGS["b"]
    eng = toy_engine(cfg, "f32", num_blocks=24, max_batch_size=2, max_tokens_per_step=48)
    w = host_weights(eng, cfg)
    prompts = [random_tokens(n, cfg["vocab"], seed=70 + n) for n in (19, 33, 8)]
    n_new = 12
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(n_new):
            toks.append(int(plain_forward(cfg, w, toks)[-1].argmax()))
        want.append(toks[len(p):])
    assert eng.generate(prompts, SamplingParams.greedy(max_tokens=n_new)) == want
