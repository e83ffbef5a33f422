"""The command line (``python -m inferrs_b200 run | bench``) on a tiny model, and the cache sized from free memory."""
import json
import os

import pytest
import torch

from helpers import CONFIG_D, random_tokens

pytestmark = pytest.mark.gpu


def test_bench_subcommand(model_dirs, capsys):
    from inferrs_b200 import cli
    rc = cli.main(["bench", model_dirs["D"], "--prompt-len", "40", "--max-tokens", "8", "--runs", "2", "--warmup", "1",
                   "--max-blocks", "64", "--max-batch-size", "2", "--temperature", "0"])
    assert rc == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["prompt_len"] == 40 and out["max_tokens"] == 8 and out["runs"] == 2
    for key in ("prefill_tok_s", "decode_tok_s", "ttft_ms", "e2e_ms_p50", "e2e_ms_p90"):
        assert out[key] > 0, key
    assert out["prefill_tok_s_sd"] >= 0 and out["decode_tok_s_sd"] >= 0


def test_run_subcommand_with_random_weights_and_prompts(tmp_path, capsys):
    """``--random-weights`` takes a config.json instead of a model folder; ``--random-prompt``, ``--prompt-file``,
    ``--ignore-eos``, ``--min-p`` and ``--prefill-chunk`` reach the engine; the same seed gives the same tokens."""
    from inferrs_b200 import cli
    cfg = dict(CONFIG_D, eos_token_id=3)
    path = str(tmp_path / "config.json")
    with open(path, "w") as f:
        json.dump(cfg, f)
    common = [path, "--random-weights", "4", "--max-blocks", "32", "--max-batch-size", "2", "--max-tokens", "6",
              "--ignore-eos", "--seed", "9", "--prefill-chunk", "16", "--dtype", "f32"]
    outs = []
    for _ in range(2):
        assert cli.main(["run"] + common + ["--random-prompt", "40", "--temperature", "0.8", "--min-p", "0.05"]) == 0
        cap = capsys.readouterr()
        outs.append([int(t) for t in cap.out.split()])
        assert "40 prompt tokens, 6 generated" in cap.err
    assert outs[0] == outs[1] and len(outs[0]) == 6
    ids_file = str(tmp_path / "prompt.txt")
    ids = random_tokens(25, cfg["vocab_size"], seed=1)
    with open(ids_file, "w") as f:
        f.write(" ".join(map(str, ids)))
    assert cli.main(["run"] + common + ["--prompt-file", ids_file, "--temperature", "0"]) == 0
    from_file = [int(t) for t in capsys.readouterr().out.split()]
    assert cli.main(["run"] + common + ["--prompt-ids", ",".join(map(str, ids)), "--temperature", "0"]) == 0
    assert from_file == [int(t) for t in capsys.readouterr().out.split()] and len(from_file) == 6
    assert cli.main(["run", path, "--random-weights", "4"]) == 2          # no prompt at all


def test_the_cache_is_sized_from_the_memory_that_is_free_once_the_model_stands():
    """Two layers of the sizes of Qwen3-8B, no number of pages given: the cache takes the asked fraction of what is
    free after the model is built and the tensors that were fused into others are given back."""
    from inferrs_b200 import Engine, SamplingParams
    from test_large_shape_gpu import CONFIG
    torch.cuda.empty_cache()
    fraction = 0.005
    eng = Engine(config=CONFIG, random_weights=1, dtype="bf16", block_size=16, num_blocks=None,
                 paged_attention=fraction, max_batch_size=64, max_seq_len=4096)
    stats = eng.stats()
    per_page = 2 * 2 * 8 * 128 * 16 * 2                      # layers x (keys, values) x heads x size x tokens x bytes
    assert stats["cache_bytes"] == stats["pages"][0] * per_page
    assert stats["pages"][0] < 64 * 256, "the fraction, not the most that the requests can use, was meant to decide"
    free_now = torch.cuda.mem_get_info()[0]
    free_before_cache = free_now + stats["cache_bytes"]     # what was free when the cache was sized, about
    assert 0.9 * fraction * free_before_cache <= stats["cache_bytes"] <= 1.02 * fraction * free_before_cache
    # the weights stand once: embedding, head, and per layer q/k/v, o, gate/up and down, nothing twice
    n_weights = 2 * 151936 * 4096 + 2 * (6144 * 4096 + 4096 * 4096 + 3 * 12288 * 4096)
    held = torch.cuda.memory_allocated() - stats["cache_bytes"]
    assert held < 2 * n_weights * 1.08, f"{held / 1e9:.2f} GB are held for {2 * n_weights / 1e9:.2f} GB of weights"
    out = eng.generate([random_tokens(50, CONFIG["vocab_size"], seed=2)], SamplingParams.greedy(max_tokens=4))
    assert len(out[0]) == 4
    del eng
    torch.cuda.empty_cache()


def test_generation_config_in_the_model_folder_ends_requests(tmp_path):
    """A model folder whose generation_config.json names an id that ends a turn: generation through the entry point
    stops there, although config.json does not name it."""
    from inferrs_b200 import Engine, SamplingParams
    from inferrs_b200.weights.random_init import write_random_model
    cfg = {k: v for k, v in CONFIG_D.items() if k != "eos_token_id"}
    folder = str(tmp_path / "model")
    write_random_model(folder, cfg, seed=12, dtype=torch.float32)
    prompt = random_tokens(30, cfg["vocab_size"], seed=2)
    kw = dict(dtype="f32", block_size=16, num_blocks=16, max_batch_size=2)
    def params(**more):     # sampled, so that the tokens differ from one another; seeded, so that they come again
        return SamplingParams(temperature=1.5, seed=5, max_tokens=10, **more)

    free = Engine(folder, **kw).generate([prompt], params())[0]
    assert len(free) == 10
    stop_at = next(i for i in range(2, 10) if free[i] not in free[:i])     # a token that has not come before
    with open(os.path.join(folder, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": [free[stop_at], cfg["vocab_size"] - 1], "temperature": 0.6}, f)
    eng = Engine(folder, **kw)
    assert free[stop_at] in eng.eos_token_ids
    assert eng.generate([prompt], params())[0] == free[:stop_at + 1]
    assert eng.generate([prompt], params(ignore_eos=True))[0] == free


def test_a_seed_gives_the_same_weights_on_the_host_and_on_the_device(tmp_path):
    """A model folder written from a seed and a model made on the device from the same seed are the same model: the
    engine gives the same logits either way, bit for bit."""
    from inferrs_b200 import Engine
    from inferrs_b200.engine.batch import StepEntry
    from inferrs_b200.parts.spec import TensorDecl
    from inferrs_b200.weights.random_init import random_tensor, write_random_model
    for init in ("normal", "norm"):
        decl = TensorDecl("a.weight", (300, 129), init=init)
        host = random_tensor(decl, 0, 11, torch.float32)
        device = random_tensor(decl, 0, 11, torch.float32, torch.device("cuda"))
        assert torch.equal(host, device.cpu())
    folder = str(tmp_path / "model")
    write_random_model(folder, CONFIG_D, seed=21, dtype=torch.bfloat16)
    toks = random_tokens(40, CONFIG_D["vocab_size"], seed=6)
    kw = dict(dtype="bf16", block_size=16, num_blocks=16, max_batch_size=2)
    logits = []
    for eng in (Engine(folder, **kw), Engine(config=CONFIG_D, random_weights=21, **kw)):
        eng.runner.admit("a")
        logits.append(eng.runner.step([StepEntry("a", toks, list(range(len(toks))))]).clone())
        eng.runner.release("a")
    assert torch.equal(logits[0], logits[1])
