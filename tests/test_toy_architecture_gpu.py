"""A whole toy architecture that only this file knows, added without a change to the package: a configuration
class, a ``build_spec`` and a mixer with state of its own, registered from here and run through the same entry
point as the real model (``Engine(config=..., random_weights=...)``).

It is no model of anyone's.  It exists to show what the descriptions can say: a scaled embedding, a layer with four
norms (one before and one after each sub-layer), a layer of a single sub-layer without a norm, soft-capped logits,
an attention layer with pages beside mixers with fixed-size state.  And it proves the state's life through the
engine's own path: a slot that is taken again starts at zero, a request that was preempted and is computed again
starts at zero, and the requests that only pad a replayed step never touch a live request's state.
"""
import math
from dataclasses import dataclass

import pytest
import torch

import plain_qwen3 as P
from helpers import random_tokens, rel_err
from inferrs_b200 import Engine, SamplingParams, kernels
from inferrs_b200.cache.storage import StateNeed
from inferrs_b200.config.base import ConfigError, RawConfig, register_architecture
from inferrs_b200.engine.batch import StepEntry
from inferrs_b200.parts import (AttentionSpec, GatedDenseSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec,
                                ScheduleEntry, SubLayerSpec, TensorDecl, pre_norm_layer, register_mixer)

pytestmark = pytest.mark.gpu

TOY_CONFIG = {
    "architectures": ["ToyStateLM"], "width": 72, "inner": 112, "vocab": 211, "heads": 4, "kv_heads": 2, "head_dim": 16,
    "theta": 5000.0, "eps": 1e-5, "positions": 256, "decay": 0.8, "embedding_scale": 3.0, "logit_scale": 0.5,
    "logit_softcap": 4.0,
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
    decay: float
    embedding_scale: float
    logit_scale: float
    logit_softcap: float

    @classmethod
    def from_raw(cls, raw: RawConfig) -> "ToyConfig":
        ints = ("width", "inner", "vocab", "heads", "kv_heads", "head_dim", "positions")
        floats = ("theta", "eps", "decay", "embedding_scale", "logit_scale", "logit_softcap")
        missing = [k for k in ints + floats if not raw.has(k)]
        if missing:
            raise ConfigError(f"{raw.source}: the toy config lacks {missing}")
        return cls(**{k: raw.get_int(k) for k in ints}, **{k: raw.get_float(k) for k in floats})


@dataclass(frozen=True)
class ToyEmaSpec:
    width: int
    decay: float
    proj: str
    kind: str = "toy_ema_rows"


class ToyEma:
    """state = decay * state + (1 - decay) * (W h), one state vector per request; the output is the state.  Written
    with device-side indexing only (no host value of the step is read), so its steps may be captured."""

    graph_safe = True

    @staticmethod
    def declare(spec):
        return [TensorDecl(spec.proj, (spec.width, spec.width))]

    @staticmethod
    def cache_need(spec):
        return None

    @staticmethod
    def state_need(spec):
        return StateNeed(shape=(spec.width,), dtype=torch.float32)

    def __init__(self, spec, weights, rt):
        self.spec, self.rt, self.w = spec, rt, weights[spec.proj].contiguous()

    def forward(self, ctx, cache_id, h):
        state = ctx.storage.state(cache_id)
        n = h.shape[0]
        u = torch.empty((n, self.spec.width), dtype=self.rt.dtype, device=h.device)
        kernels.linear(h, self.w, u, self.rt.dtype)
        u = u.float()
        row_slot = ctx.slots.long().index_select(0, ctx.row_request.long())
        out = torch.empty_like(u)
        d = self.spec.decay
        for r in range(n):                       # the rows of a request stand together, in order
            idx = row_slot[r:r + 1]
            s = state.index_select(0, idx) * d + (1.0 - d) * u[r:r + 1]
            state.index_copy_(0, idx, s)
            out[r:r + 1] = s
        return out.to(h.dtype)


def build_toy_spec(cfg: ToyConfig) -> ModelSpec:
    def norm(name):
        return NormSpec(size=cfg.width, eps=cfg.eps, weight=name)

    def dense(p):
        return GatedDenseSpec(width=cfg.width, inner=cfg.inner, gate_proj=f"{p}.gate_proj.weight",
                              up_proj=f"{p}.up_proj.weight", down_proj=f"{p}.down_proj.weight")

    position = PositionSpec(kind="rotary_split_half", rot_dim=cfg.head_dim, theta=cfg.theta, max_positions=cfg.positions)
    a = "blocks.0.attn"
    attention = AttentionSpec(
        width=cfg.width, n_heads=cfg.heads, n_kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
        scale=1.0 / math.sqrt(cfg.head_dim), position=position, q_proj=f"{a}.q_proj.weight",
        k_proj=f"{a}.k_proj.weight", v_proj=f"{a}.v_proj.weight", o_proj=f"{a}.o_proj.weight",
        q_norm=NormSpec(size=cfg.head_dim, eps=cfg.eps, weight=f"{a}.q_norm.weight"),
        k_norm=NormSpec(size=cfg.head_dim, eps=cfg.eps, weight=f"{a}.k_norm.weight"))
    layers = (
        # a pre-norm block of attention and a gated feed-forward
        pre_norm_layer(norm("blocks.0.n1.weight"), attention, norm("blocks.0.n2.weight"), dense("blocks.0.mlp")),
        # four norms: one before and one after each sub-layer
        LayerSpec(sublayers=(
            SubLayerSpec(part=ToyEmaSpec(cfg.width, cfg.decay, "blocks.1.ema.weight"), category="mixer",
                         norm=norm("blocks.1.pre_mixer.weight"), post_norm=norm("blocks.1.post_mixer.weight")),
            SubLayerSpec(part=dense("blocks.1.mlp"), category="feed_forward",
                         norm=norm("blocks.1.pre_ffn.weight"), post_norm=norm("blocks.1.post_ffn.weight")))),
        # a single sub-layer that reads the residual stream as it is
        LayerSpec(sublayers=(
            SubLayerSpec(part=ToyEmaSpec(cfg.width, cfg.decay, "blocks.2.ema.weight"), category="mixer"),)),
    )
    return ModelSpec(
        vocab_size=cfg.vocab, width=cfg.width, embedding="emb.weight", layers=layers,
        schedule=tuple(ScheduleEntry(layer=i, cache=i) for i in range(len(layers))),
        final_norm=norm("final.weight"), lm_head="head.weight", lm_head_optional=False, max_positions=cfg.positions,
        embedding_scale=cfg.embedding_scale, logit_scale=cfg.logit_scale, logit_softcap=cfg.logit_softcap,
        architecture="ToyStateLM")


def register_toy():
    register_mixer("toy_ema_rows", ToyEma, replace=True)
    register_architecture("ToyStateLM", ToyConfig, build_toy_spec, replace=True)


def plain_toy_forward(c: dict, w: dict, ids) -> torch.Tensor:
    """The toy as whole-sequence arithmetic in float32: logits of every position."""
    def ema(x, weight):
        u = x @ weight.t()
        s, out = torch.zeros(x.shape[1]), []
        for t in range(x.shape[0]):
            s = c["decay"] * s + (1.0 - c["decay"]) * u[t]
            out.append(s)
        return torch.stack(out)

    t = len(ids)
    x = P.embedding(torch.tensor(ids), w["emb.weight"]) * c["embedding_scale"]
    acfg = {"num_attention_heads": c["heads"], "num_key_value_heads": c["kv_heads"], "head_dim": c["head_dim"],
            "rms_norm_eps": c["eps"]}
    cos, sin = P.rope_tables(c["head_dim"], c["theta"], t, torch.float32)
    x = x + P.attention_layer(P.rms_norm(x, w["blocks.0.n1.weight"], c["eps"]), w, "blocks.0.attn", acfg, cos, sin)
    x = x + P.mlp(P.rms_norm(x, w["blocks.0.n2.weight"], c["eps"]), w, "blocks.0.mlp")
    y = ema(P.rms_norm(x, w["blocks.1.pre_mixer.weight"], c["eps"]), w["blocks.1.ema.weight"])
    x = x + P.rms_norm(y, w["blocks.1.post_mixer.weight"], c["eps"])
    y = P.mlp(P.rms_norm(x, w["blocks.1.pre_ffn.weight"], c["eps"]), w, "blocks.1.mlp")
    x = x + P.rms_norm(y, w["blocks.1.post_ffn.weight"], c["eps"])
    x = x + ema(x, w["blocks.2.ema.weight"])
    logits = P.linear(P.rms_norm(x, w["final.weight"], c["eps"]), w["head.weight"]) * c["logit_scale"]
    return c["logit_softcap"] * torch.tanh(logits / c["logit_softcap"])


def toy_engine(**kw) -> Engine:
    register_toy()
    eng = Engine(config=TOY_CONFIG, random_weights=17, dtype="f32", block_size=16, **kw)
    # the mixers' projections larger, so that the state decides the logits
    for blk in eng.runner.model.blocks[1:]:
        for p in blk.parts():
            if isinstance(p, ToyEma):
                p.w.mul_(8.0)
    eng.runner.model.head.weight.mul_(40.0)     # and logits large enough for the cap to bend them
    return eng


def host_weights(eng: Engine) -> dict:
    m = eng.runner.model
    w = {"emb.weight": m.embedding, "head.weight": m.head.weight, "final.weight": m.final_norm.weight}
    a = m.blocks[0].sublayers[0].part
    nh, nkv, d = TOY_CONFIG["heads"], TOY_CONFIG["kv_heads"], TOY_CONFIG["head_dim"]
    q, k, v = a.qkv.weight.split([nh * d, nkv * d, nkv * d])
    w.update({"blocks.0.attn.q_proj.weight": q, "blocks.0.attn.k_proj.weight": k, "blocks.0.attn.v_proj.weight": v,
              "blocks.0.attn.o_proj.weight": a.o.weight, "blocks.0.attn.q_norm.weight": a.q_weight,
              "blocks.0.attn.k_norm.weight": a.k_weight})
    for b, names in ((0, ("n1", "n2")), (1, ("pre_mixer", "pre_ffn"))):
        for s, name in zip(m.blocks[b].sublayers, names):
            w[f"blocks.{b}.{name}.weight"] = s.norm.weight
    for s, name in zip(m.blocks[1].sublayers, ("post_mixer", "post_ffn")):
        w[f"blocks.1.{name}.weight"] = s.post_norm.weight
    for b, sub in ((0, 1), (1, 1)):
        f = m.blocks[b].sublayers[sub].part
        g, u = f.gate_up.weight.split([TOY_CONFIG["inner"], TOY_CONFIG["inner"]])
        w.update({f"blocks.{b}.mlp.gate_proj.weight": g, f"blocks.{b}.mlp.up_proj.weight": u,
                  f"blocks.{b}.mlp.down_proj.weight": f.down.weight})
    w["blocks.1.ema.weight"] = m.blocks[1].sublayers[0].part.w
    w["blocks.2.ema.weight"] = m.blocks[2].sublayers[0].part.w
    return {k: t.float().cpu() for k, t in w.items()}


def plain_greedy(w: dict, prompt, n: int):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(plain_toy_forward(TOY_CONFIG, w, toks)[-1].argmax()))
    return toks[len(prompt):]


def test_toy_architecture_is_registered_built_and_stepped_like_its_plain_statement():
    eng = toy_engine(num_blocks=32, max_batch_size=3, max_tokens_per_step=64)
    runner = eng.runner
    assert runner.graphs is not None, "every part of the toy says graph_safe: its steps are replayed graphs"
    assert sorted(runner.storage.states) == [1, 2] and len(runner.storage.kv) == 1
    w = host_weights(eng)
    toks = random_tokens(75, TOY_CONFIG["vocab"], seed=3)
    want = plain_toy_forward(TOY_CONFIG, w, toks)
    assert float(want.abs().max()) < TOY_CONFIG["logit_softcap"] and float(want.abs().max()) > 1.0
    # whole, and in portions of changing size with a second request's tokens beside them
    other = random_tokens(40, TOY_CONFIG["vocab"], seed=4)
    runner.admit("whole")
    got = runner.step([StepEntry("whole", toks, list(range(len(toks))))])
    assert rel_err(got, want) < 1e-4
    runner.release("whole")
    runner.admit("cut")
    runner.admit("other")
    at, rows, o_at = 0, [], 0
    for n in (7, 2, 30, 1, 1, 20, 3, 11):
        entries = [StepEntry("cut", toks[at:at + n], list(range(n)))]
        if o_at < len(other):
            entries.append(StepEntry("other", other[o_at:o_at + 6], []))
            o_at += 6
        rows.append(runner.step(entries)[:n])
        at += n
    assert at == len(toks)
    assert rel_err(torch.cat(rows), want) < 1e-4


def test_state_is_fresh_for_every_admission_through_generate():
    """More requests than slots, and so few pages that a request is preempted and computed again: every request
    still gets the tokens of the plain statement, which knows no slots."""
    eng = toy_engine(num_blocks=7, max_batch_size=2, max_tokens_per_step=48)
    w = host_weights(eng)
    prompts = [random_tokens(n, TOY_CONFIG["vocab"], seed=50 + n) for n in (33, 21, 40, 9, 27)]
    n_new = 30
    want = [plain_greedy(w, p, n_new) for p in prompts]
    got = eng.generate(prompts, SamplingParams.greedy(max_tokens=n_new))
    stats = eng.stats()
    assert stats["preemptions"] > 0, "the cache was meant to be too small for two requests to finish side by side"
    assert stats["steps_ahead"] > 0, "steps were meant to be replayed graphs launched one ahead"
    eng.runner.manager.check_invariants()
    assert got == want
    # a second round on the same engine: every slot has had an occupant before
    again = eng.generate(prompts[:3], SamplingParams.greedy(max_tokens=n_new))
    assert again == want[:3]
