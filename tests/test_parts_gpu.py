"""Each part alone against the plain functions, and the generality of their assembly: layers with
different mixers, a window group whose pages come back early, a layer that runs twice, a layer that
reads another layer's cache, and a toy mixer with state of its own that only this file knows."""
import dataclasses
from dataclasses import dataclass
from typing import Optional

import pytest
import torch

import plain_qwen3 as P
from helpers import CONFIG_B, CONFIG_C, cut, random_tokens, rel_err
from inferrs_b200.cache.manager import RELEASED, CacheManager
from inferrs_b200.cache.storage import CacheStorage, KVNeed, StateNeed
from inferrs_b200.engine.batch import StepEntry, build_context
from inferrs_b200.engine.loading import spec_from_config
from inferrs_b200.engine.model import declared_tensors
from inferrs_b200.engine.runner import ModelRunner
from inferrs_b200.parts import (AttentionSpec, GatedDenseSpec, LayerSpec, NormSpec, PositionSpec, ScheduleEntry,
                                TensorDecl, part_class, register_mixer)
from inferrs_b200.runtime import Runtime
from inferrs_b200.weights.random_init import random_weights

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def weights_for(decls, dtype, seed=0):
    w = random_weights(decls, seed, torch.bfloat16)            # values that bfloat16 holds exactly
    return {k: v.to(dtype).cuda() for k, v in w.items()}


def one_request_ctx(kv_need: Optional[KVNeed], n_tokens, start, dtype, page_size=16, state_needs=None):
    """A step context for one request that already holds `start` tokens and brings `n_tokens` more."""
    storage = CacheStorage({0: kv_need} if kv_need else {}, state_needs or {}, page_size, 64, 2, dtype,
                           torch.device("cuda"))
    manager = CacheManager(storage.layouts, page_size, storage.n_pages, 2)
    manager.admit("r")
    if start:
        manager.reserve({"r": start})
        manager.commit("r", start)
    manager.reserve({"r": n_tokens})
    ctx = build_context([StepEntry("r", [1] * n_tokens, [])], manager, storage, 10, 4096, torch.device("cuda"))
    return ctx, storage, manager


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(dtype):
    rt = Runtime.cuda(dtype)
    spec = NormSpec(size=200, eps=1e-5, weight="n.weight")
    cls = part_class("norm", spec)
    assert [(d.name, d.shape, d.init) for d in cls.declare(spec)] == [("n.weight", (200,), "norm")]
    w = weights_for(cls.declare(spec), dtype)
    part = cls(spec, w, rt)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(7, 200, generator=g)
    delta = torch.randn(7, 200, generator=g).to(dtype)
    res = x.clone().cuda()
    out = part.add_norm(res, delta.cuda())
    want_x = x + delta.float()
    assert rel_err(res.cpu(), want_x) < 1e-6
    assert rel_err(out.float().cpu(), P.rms_norm(want_x, w["n.weight"].float().cpu(), 1e-5)) < TOL[dtype]


def test_rotary_tables_part():
    rt = Runtime.cuda(torch.float32)
    spec = PositionSpec(kind="rotary_split_half", rot_dim=48, theta=50000.0, max_positions=300)
    cos, sin, rot = part_class("position", spec)(spec, rt).tables()
    pc, ps = P.rope_tables(48, 50000.0, 300, torch.float32)
    assert rot == 48 and torch.allclose(cos.cpu(), pc, atol=1e-6) and torch.allclose(sin.cpu(), ps, atol=1e-6)
    assert part_class("position", PositionSpec(kind="none"))(PositionSpec(kind="none"), rt).tables()[2] == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part(dtype, window):
    rt = Runtime.cuda(dtype)
    nh, nkv, d, width, t = 6, 2, 64, 80, 50
    spec = AttentionSpec(width=width, n_heads=nh, n_kv_heads=nkv, head_dim=d, scale=d ** -0.5,
                         position=PositionSpec(rot_dim=d, theta=10000.0, max_positions=256),
                         q_proj="a.q_proj.weight", k_proj="a.k_proj.weight", v_proj="a.v_proj.weight",
                         o_proj="a.o_proj.weight", q_norm=NormSpec(d, 1e-6, "a.q_norm.weight"),
                         k_norm=NormSpec(d, 1e-6, "a.k_norm.weight"), window=window)
    cls = part_class("mixer", spec)
    assert cls.cache_need(spec) == KVNeed(nkv, d, window) and cls.state_need(spec) is None
    w = weights_for(cls.declare(spec), dtype, seed=3)
    for k in w:
        if "proj" in k:
            w[k] = (w[k].float() * 5).to(dtype)   # scores that are not all alike
    part = cls(spec, w, rt)
    h = (torch.randn(t, width, generator=torch.Generator().manual_seed(1))).to(dtype)
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": d, "rms_norm_eps": 1e-6}
    cos, sin = P.rope_tables(d, 10000.0, t, torch.float32)
    store = None if dtype == torch.float32 else dtype
    want = P.attention_layer(h.float(), {k: v.float().cpu() for k, v in w.items()}, "a", cfg, cos, sin, store, window)
    # whole, then the same rows as a portion of 37 and 13 single steps on a fresh cache
    ctx, _, _ = one_request_ctx(cls.cache_need(spec), t, 0, dtype)
    got = part.forward(ctx, 0, h.cuda())
    assert rel_err(got.float().cpu(), want) < TOL[dtype]
    storage = CacheStorage({0: cls.cache_need(spec)}, {}, 16, 64, 2, dtype, torch.device("cuda"))
    manager = CacheManager(storage.layouts, 16, storage.n_pages, 2)
    manager.admit("r")
    rows, at = [], 0
    for n in [37] + [1] * 13:
        manager.reserve({"r": n})
        ctx = build_context([StepEntry("r", [1] * n, [])], manager, storage, 10, 4096, torch.device("cuda"))
        rows.append(part.forward(ctx, 0, h[at:at + n].cuda()))
        manager.commit("r", n)
        at += n
    assert rel_err(torch.cat(rows).float().cpu(), want) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_dense_part(dtype):
    rt = Runtime.cuda(dtype)
    spec = GatedDenseSpec(width=72, inner=200, gate_proj="m.gate_proj.weight", up_proj="m.up_proj.weight",
                          down_proj="m.down_proj.weight")
    cls = part_class("feed_forward", spec)
    w = weights_for(cls.declare(spec), dtype, seed=4)
    w = {k: (v.float() * 10).to(dtype) for k, v in w.items()}
    part = cls(spec, w, rt)
    h = torch.randn(9, 72, generator=torch.Generator().manual_seed(2)).to(dtype)
    want = P.mlp(h.float(), {k: v.float().cpu() for k, v in w.items()}, "m",
                 None if dtype == torch.float32 else dtype)
    assert rel_err(part.forward(None, h.cuda()).float().cpu(), want) < TOL[dtype]
    with pytest.raises(ValueError, match="activation"):
        cls(dataclasses.replace(spec, activation="gelu"), w, rt)


# ---- assemblies that the architecture itself does not use --------------------------------------------

def plain_scheduled(cfg, w, ids, schedule, windows, store=None):
    """The plain decoder with layers run in `schedule` order (a layer may come twice) and per-layer windows."""
    w = {k: v.float() for k, v in w.items()}
    cos, sin = P.rope_tables(cfg["head_dim"], cfg["rope_theta"], len(ids), torch.float32)
    x = P.embedding(torch.tensor(ids), w["model.embed_tokens.weight"])
    for layer in schedule:
        x = P.decoder_layer(x, w, layer, cfg, cos, sin, store, windows[layer])
    x = P._rnd(P.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]), store)
    return P.linear(x, w.get("lm_head.weight", w["model.embed_tokens.weight"]))


def run_cut(runner, rid, toks, sizes):
    runner.admit(rid)
    rows, at = [], 0
    for n in cut(len(toks), sizes):
        rows.append(runner.step([StepEntry(rid, toks[at:at + n], list(range(n)))]))
        at += n
    return torch.cat(rows)


@pytest.mark.parametrize("dtype,cfg", [(torch.float32, CONFIG_B), (torch.bfloat16, CONFIG_C)])
def test_layers_with_different_mixers_windows_and_a_layer_twice(dtype, cfg):
    spec, _ = spec_from_config(cfg)
    layers = list(spec.layers)
    layers[1] = layers[1].with_part("mixer", dataclasses.replace(layers[1].mixer, window=24))
    order = [0, 1, 1] + list(range(2, len(layers)))
    spec = dataclasses.replace(spec, layers=tuple(layers),
                               schedule=tuple(ScheduleEntry(layer=l, cache=i) for i, l in enumerate(order)))
    rt = Runtime.cuda(dtype)
    weights = weights_for(declared_tensors(spec), dtype, seed=6)
    runner = ModelRunner(spec, weights, rt, page_size=16, n_pages=24, max_requests=4)
    assert len(runner.storage.kv) == 2 and sorted(l.window or 0 for l in runner.storage.layouts) == [0, 24]
    toks = random_tokens(150, cfg["vocab_size"], seed=3)
    windows = [24 if i == 1 else None for i in range(len(layers))]
    want = plain_scheduled(cfg, {k: v.cpu() for k, v in weights.items()}, toks, order, windows,
                           None if dtype == torch.float32 else dtype)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert rel_err(run_cut(runner, "whole", toks, [150]).cpu(), want) < tol
    runner.release("whole")
    got = run_cut(runner, "cut", toks, [7, 2, 40, 1, 1, 19, 3])
    assert rel_err(got.cpu(), want) < tol
    # the window group has given back the pages that its window has passed; the full group holds all
    g_win = next(g for g, l in enumerate(runner.storage.layouts) if l.window == 24)
    table = runner.manager.block_table("cut", g_win)
    assert sum(p != RELEASED for p in table) <= 3 and sum(p == RELEASED for p in table) >= 7
    assert all(p != RELEASED for p in runner.manager.block_table("cut", 1 - g_win))
    runner.manager.check_invariants()


def test_a_layer_that_reads_another_layers_cache():
    cfg, dtype = CONFIG_C, torch.float32
    spec, _ = spec_from_config(cfg)
    layers = list(spec.layers)
    reader = dataclasses.replace(layers[1].mixer, own_kv=False, k_proj=None, v_proj=None, k_norm=None)
    layers[1] = layers[1].with_part("mixer", reader)
    spec = dataclasses.replace(spec, layers=tuple(layers), schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 0)))
    names = [d.name for d in declared_tensors(spec)]
    assert "model.layers.1.self_attn.k_proj.weight" not in names
    rt = Runtime.cuda(dtype)
    runner = ModelRunner(spec, weights_for(declared_tensors(spec), dtype, seed=8), rt, page_size=16, n_pages=16,
                         max_requests=2)
    assert runner.storage.kv[0].shape[0] == 1       # one cache serves both entries
    toks = random_tokens(70, cfg["vocab_size"], seed=4)
    whole = run_cut(runner, "a", toks, [70])
    parts = run_cut(runner, "b", toks, [9, 2, 30, 1, 1, 1])
    assert rel_err(parts, whole) < 1e-4


# ---- a toy mixer with state of its own, known only to this file ---------------------------------------

@dataclass(frozen=True)
class ToyEmaSpec:
    """y_t = s_t,  s_t = decay * s_{t-1} + (1 - decay) * (h_t W^T): a running mean that needs the state of the
    request's earlier tokens, of fixed size, and no pages."""
    width: int
    decay: float
    proj: str
    kind: str = "toy_ema"


class ToyEma:
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
        self.spec, self.rt, self.w = spec, rt, weights[spec.proj].float()

    def forward(self, ctx, cache_id, h):
        state = ctx.storage.state(cache_id)
        u = h.float() @ self.w.t()
        out = torch.empty_like(u)
        row = 0
        for slot, n in zip(ctx.slot_list, ctx.q_lens):      # the rows of a request stand together, in order
            s = state[slot].clone()
            for t in range(n):
                s = self.spec.decay * s + (1.0 - self.spec.decay) * u[row]
                out[row] = s
                row += 1
            state[slot] = s
        return out.to(h.dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype):
    register_mixer("toy_ema", ToyEma, replace=True)
    cfg = CONFIG_C
    spec, _ = spec_from_config(cfg)
    layers = list(spec.layers)
    toy = ToyEmaSpec(width=cfg["hidden_size"], decay=0.8, proj="model.layers.1.toy.proj.weight")
    layers[1] = layers[1].with_part("mixer", toy)
    spec = dataclasses.replace(spec, layers=tuple(layers))
    names = [d.name for d in declared_tensors(spec)]
    assert toy.proj in names and "model.layers.1.self_attn.q_proj.weight" not in names
    rt = Runtime.cuda(dtype)
    weights = weights_for(declared_tensors(spec), dtype, seed=9)
    weights[toy.proj] = (weights[toy.proj].float() * 20).to(dtype)
    runner = ModelRunner(spec, weights, rt, page_size=16, n_pages=32, max_requests=3)
    assert runner.graphs is None, "a part that does not declare graph_safe must keep the step out of CUDA graphs"
    assert list(runner.storage.states) == [1] and runner.storage.states[1].shape == (3 + 1, cfg["hidden_size"])   # one more for padding requests
    assert len(runner.storage.kv) == 1 and runner.storage.kv[0].shape[0] == 1   # only layer 0 has pages
    toks = [random_tokens(n, cfg["vocab_size"], seed=20 + n) for n in (60, 45, 33)]
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    whole = []
    for i, t in enumerate(toks):
        whole.append(run_cut(runner, ("w", i), t, [len(t)]))
        runner.release(("w", i))
    # portions, then decoding, with the three requests side by side: the state is carried between steps
    for i in range(3):
        runner.admit(("m", i))
    at, got = [0, 0, 0], [[], [], []]
    sizes = [[7, 2, 30, 1], [1, 1, 20, 3], [33]]
    step = 0
    while any(at[i] < len(toks[i]) for i in range(3)):
        entries = []
        for i in range(3):
            if at[i] < len(toks[i]):
                n = min(sizes[i][step % len(sizes[i])], len(toks[i]) - at[i])
                entries.append((i, n))
        out = runner.step([StepEntry(("m", i), toks[i][at[i]:at[i] + n], list(range(n))) for i, n in entries])
        o = 0
        for i, n in entries:
            got[i].append(out[o:o + n])
            o += n
            at[i] += n
        step += 1
    for i in range(3):
        assert rel_err(torch.cat(got[i]), whole[i]) < tol, i
    # a slot that is taken again starts from a cleared state
    runner.release(("m", 0))
    again = run_cut(runner, "again", toks[0], [len(toks[0])])
    assert rel_err(again, whole[0]) < (1e-6 if dtype == torch.float32 else tol)
    # and the state matters: without the earlier tokens the later logits differ
    runner.release("again")
    tail = run_cut(runner, "tail", toks[0][30:], [30])
    assert rel_err(tail, whole[0][30:]) > 10 * tol


def test_replayed_steps_get_the_description_that_the_general_builder_gives():
    """Decode steps are replayed graphs whose description native code writes from the cache's book: after
    every step it must equal what the general builder gives for the same entries, across page edges, with a
    window group that gives pages back, and when requests come and go."""
    import numpy as np
    from inferrs_b200.engine.batch import build_context
    spec, _ = spec_from_config(CONFIG_B)
    layers = list(spec.layers)
    layers[1] = layers[1].with_part("mixer", dataclasses.replace(layers[1].mixer, window=24))
    spec = dataclasses.replace(spec, layers=tuple(layers))
    rt = Runtime.cuda(torch.float32)
    weights = weights_for(declared_tensors(spec), torch.float32, seed=8)
    runner = ModelRunner(spec, weights, rt, page_size=16, n_pages=40, max_requests=4)
    dg = runner.graphs
    assert dg is not None
    checked_steps = []
    original = dg._describe

    def checked(cap, entries, bucket, carry=None):
        turn = cap.turn
        original(cap, entries, bucket, carry)
        ctx = build_context(entries, runner.manager, runner.storage, spec.vocab_size, spec.max_positions,
                            torch.device("cpu"), fixed_pages=dg.fixed_pages, pad_to=bucket)
        host = ctx.extra["host"]
        torch.cuda.synchronize()
        assert np.array_equal(cap.staging[turn].numpy()[:host.size], host)
        assert np.array_equal(cap.buffer.cpu().numpy()[:host.size], host)
        checked_steps.append(len(entries))

    dg._describe = checked
    vocab = CONFIG_B["vocab_size"]
    for rid, n in (("a", 13), ("b", 30), ("c", 47)):
        runner.admit(rid)
        runner.step([StepEntry(rid, random_tokens(n, vocab, seed=n), [])])
    live = ["a", "b", "c"]
    for step in range(70):
        if step == 25:
            runner.release("b")
            live.remove("b")
        if step == 40:
            runner.admit("d")
            runner.step([StepEntry("d", random_tokens(5, vocab, seed=5), [])])
            live.append("d")
        runner.step([StepEntry(rid, [(7 * step + i) % vocab], [0]) for i, rid in enumerate(live)])
    assert len(checked_steps) > 60 and set(checked_steps) == {2, 3}
    runner.manager.check_invariants()
