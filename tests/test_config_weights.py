"""Configuration, registry and weight loading: what is read, what is refused, and how it is said."""
import json
import os

import pytest
import torch

from helpers import CONFIG_A, CONFIG_B
from inferrs_b200.config import ConfigError, Qwen3Config, RawConfig, registered_architectures, resolve_architecture
from inferrs_b200.engine.loading import spec_from_config
from inferrs_b200.engine.model import declared_tensors
from inferrs_b200.weights.loader import WeightError, load_weights
from inferrs_b200.weights.random_init import write_random_model
from inferrs_b200.weights.safetensors_io import SafetensorsFile, write_safetensors


def test_registry_resolves_by_architecture_then_model_type():
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert resolve_architecture(RawConfig(CONFIG_A)).name == "Qwen3ForCausalLM"
    only_type = {k: v for k, v in CONFIG_A.items() if k != "architectures"}
    assert resolve_architecture(RawConfig(only_type)).name == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError, match="unsupported model architecture.*registered"):
        resolve_architecture(RawConfig({"architectures": ["Qwen3_5ForCausalLM"], "model_type": "qwen3_5"}))


def test_typed_config_reads_every_key():
    for c in (CONFIG_A, CONFIG_B):
        cfg = Qwen3Config.from_raw(RawConfig(c))
        assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers) == \
            (c["vocab_size"], c["hidden_size"], c["intermediate_size"], c["num_hidden_layers"])
        assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == \
            (c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"])
        assert cfg.rms_norm_eps == c["rms_norm_eps"] and cfg.rope_theta == c["rope_theta"]
        assert Qwen3Config.from_raw(RawConfig(cfg.to_dict())) == cfg


def test_head_dim_defaults_to_hidden_over_heads():
    c = {k: v for k, v in CONFIG_A.items() if k != "head_dim"}
    assert Qwen3Config.from_raw(RawConfig(c)).head_dim == 16


@pytest.mark.parametrize("change,match", [
    ({"num_key_value_heads": 3}, "not a multiple"),
    ({"hidden_size": None}, "lacks the keys"),
    ({"rope_theta": None}, "lacks the keys"),
    ({"vocab_size": "many"}, "must be an integer"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"use_sliding_window": True}, "sliding"),
    ({"eos_token_id": 100000}, "outside the vocabulary"),
])
def test_config_refusals(change, match):
    c = dict(CONFIG_A)
    c.update(change)
    with pytest.raises(ConfigError, match=match):
        Qwen3Config.from_raw(RawConfig(c))


def test_spec_holds_the_configuration_layer_by_layer():
    spec, cfg = spec_from_config(CONFIG_B)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    a = spec.layers[1].mixer
    assert (a.n_heads, a.n_kv_heads, a.head_dim, a.window) == (8, 2, 32, None)
    assert a.position.theta == 1e6 and a.position.rot_dim == 32 and a.q_norm.eps == 1e-5
    assert spec.layers[2].ffn.inner == 272 and not spec.lm_head_optional
    names = [d.name for d in declared_tensors(spec)]
    assert len(names) == len(set(names)) == 3 * 11 + 3
    assert "model.layers.2.self_attn.k_norm.weight" in names and "lm_head.weight" in names


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
         "c": torch.randn(2, 2, 2)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t.items())
    f = SafetensorsFile(p)
    for k, v in t.items():
        assert torch.equal(f.read(k), v) and f.read(k).dtype == v.dtype
    from safetensors import safe_open
    with safe_open(p, framework="pt") as g:   # the library reads what we wrote
        assert torch.equal(g.get_tensor("a"), t["a"])
    f.close()


def _decls(cfg):
    return declared_tensors(spec_from_config(cfg)[0])


def test_load_keeps_stored_precision(tmp_path):
    d = write_random_model(str(tmp_path / "m"), CONFIG_A, seed=0, dtype=torch.bfloat16)
    w = load_weights(d, _decls(CONFIG_A), torch.bfloat16)
    assert all(t.dtype == torch.bfloat16 for t in w.values()) and "lm_head.weight" not in w
    w32 = load_weights(d, _decls(CONFIG_A), torch.float32)
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert torch.equal(w32["model.norm.weight"], w["model.norm.weight"].float())
    d2 = write_random_model(str(tmp_path / "m32"), CONFIG_A, seed=0, dtype=torch.float32)
    w = load_weights(d2, _decls(CONFIG_A), torch.bfloat16)
    assert all(t.dtype == torch.float32 for t in w.values()), "a tensor stored in 32-bit stays so"


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(str(tmp_path / "m"), CONFIG_B, seed=1)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.read(n) for n in f.info}
    f.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.ones(31, dtype=torch.bfloat16)
    tensors["model.layers.7.extra.weight"] = torch.ones(2)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    with pytest.raises(WeightError) as e:
        load_weights(d, _decls(CONFIG_B), torch.float32)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "lm_head.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert len(err.wrong_shape) == 1 and "expected [32], found [31]" in err.wrong_shape[0]
    for part in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)"):
        assert part in str(err)


def test_random_weights_are_seeded(tmp_path):
    a = write_random_model(str(tmp_path / "a"), CONFIG_A, seed=3)
    b = write_random_model(str(tmp_path / "b"), CONFIG_A, seed=3)
    c = write_random_model(str(tmp_path / "c"), CONFIG_A, seed=4)
    rd = lambda d: open(os.path.join(d, "model.safetensors"), "rb").read()  # noqa: E731
    assert rd(a) == rd(b) != rd(c)
    assert json.load(open(os.path.join(a, "config.json"))) == CONFIG_A
    w = load_weights(a, _decls(CONFIG_A), torch.float32)
    assert abs(float(w["model.embed_tokens.weight"].std()) - 0.02) < 0.002
    n = w["model.layers.0.input_layernorm.weight"]
    assert 0.9 <= float(n.min()) and float(n.max()) <= 1.1 and float(n.std()) > 0.01
    # a value depends on the seed, the tensor's name and the element's index only: not on the tensor's place in the
    # declaration, and not on how many elements are made at a time
    from inferrs_b200.parts.spec import TensorDecl
    from inferrs_b200.weights import random_init
    decl = TensorDecl("some.weight", (37, 53))
    one = random_init.random_tensor(decl, 0, 9, torch.float32)
    assert torch.equal(one, random_init.random_tensor(decl, 5, 9, torch.float32))
    whole = random_init._CHUNK
    try:
        random_init._CHUNK = 100
        assert torch.equal(one, random_init.random_tensor(decl, 0, 9, torch.float32))
    finally:
        random_init._CHUNK = whole
    other = random_init.random_tensor(TensorDecl("some.other.weight", (37, 53)), 0, 9, torch.float32)
    assert abs(float((one * other).mean()) / float(one.std() * other.std())) < 0.1


def test_sharded_files_later_wins(tmp_path):
    d = write_random_model(str(tmp_path / "m"), CONFIG_A, seed=0)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.read(n) for n in f.info}
    f.close()
    os.remove(os.path.join(d, "model.safetensors"))
    names = sorted(tensors)
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), [(n, tensors[n]) for n in names[:10]])
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), [(n, tensors[n]) for n in names[8:]])
    w = load_weights(d, _decls(CONFIG_A), torch.bfloat16)
    assert all(torch.equal(w[n], tensors[n]) for n in names)


def test_generation_config_names_more_ids_that_end_a_request(tmp_path):
    from inferrs_b200.config.base import ConfigError, generation_eos_ids
    d = str(tmp_path)
    assert generation_eos_ids(d, 100) == ()                       # no such file
    (tmp_path / "generation_config.json").write_text('{"temperature": 0.6}')
    assert generation_eos_ids(d, 100) == ()                       # no such key
    (tmp_path / "generation_config.json").write_text('{"eos_token_id": 7}')
    assert generation_eos_ids(d, 100) == (7,)
    (tmp_path / "generation_config.json").write_text('{"eos_token_id": [7, 45]}')
    assert generation_eos_ids(d, 100) == (7, 45)
    for bad in ('{"eos_token_id": [7, 100]}', '{"eos_token_id": "7"}', '{"eos_token_id": [true]}', '{"eos_token_id": '):
        (tmp_path / "generation_config.json").write_text(bad)
        with pytest.raises(ConfigError):
            generation_eos_ids(d, 100)


def test_tensors_written_one_at_a_time_and_read_as_views(tmp_path):
    """The writer that makes tensors as their turn comes writes the same file as the one that is handed all of them,
    and refuses a tensor that is not what was announced; a view of the mapped file reads the same values as a copy."""
    from inferrs_b200.weights.safetensors_io import SafetensorsError, write_safetensors_streamed
    g = torch.Generator().manual_seed(3)
    tensors = {"a": torch.randn((5, 7), generator=g).to(torch.bfloat16), "b": torch.arange(12, dtype=torch.int32).view(3, 4),
               "c": torch.randn((9,), generator=g)}
    whole, streamed = str(tmp_path / "whole.safetensors"), str(tmp_path / "streamed.safetensors")
    write_safetensors(whole, tensors.items(), metadata={"k": "v"})
    made = []
    entries = [(n, tuple(t.shape), t.dtype, (lambda n=n, t=t: made.append(n) or t)) for n, t in tensors.items()]
    write_safetensors_streamed(streamed, entries, metadata={"k": "v"})
    assert made == ["a", "b", "c"]
    assert open(whole, "rb").read() == open(streamed, "rb").read()
    f = SafetensorsFile(streamed)
    for n, t in tensors.items():
        view = f.read(n, private=False)
        assert torch.equal(view, t) and torch.equal(f.read(n), t)
        del view
    f.close()
    with pytest.raises(SafetensorsError, match="announced"):
        write_safetensors_streamed(streamed, [("a", (5, 8), torch.bfloat16, lambda: tensors["a"])])

