"""Command line and recipes: plan mode, precedence, refusals."""

import os

import pytest

from sllm_b200.config import ConfigError
from sllm_b200.config.recipe import Recipe, resolve_recipe
from sllm_b200.serving import main as cli

RECIPES = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "recipes")


def test_shipped_recipe_loads():
    r = resolve_recipe("Qwen2.5-Coder-0.5B", RECIPES)
    cfg = r.config_json()
    assert (cfg["num_hidden_layers"], cfg["hidden_size"], cfg["head_dim"], cfg["rope_theta"]) == (24, 896, 64, 1e6)
    assert cfg["tie_word_embeddings"] is True and r.arch == "qwen2" and r.defaults["max_num_seqs"] == 8
    from sllm_b200.models.qwen2 import Qwen2Config
    assert Qwen2Config.from_dict(cfg).num_key_value_heads == 2


@pytest.mark.parametrize("raw,word", [
    ({"model_id": "x"}, "arch"), ({"arch": "llama4", "model_id": "x"}, "not served"),
    ({"arch": "qwen2", "model_id": "x", "dtype": "fp8"}, "dtype"),
    ({"arch": "qwen2", "model_id": "x", "tp": {"size": 2}}, "one GPU"),
    ({"arch": "qwen2", "model_id": "x", "defaults": {"max_new": 0}}, "max_new"),
    ({"arch": "qwen2", "model_id": "x", "memory": {"kv_utilization": 1.5}}, "kv_utilization"),
])
def test_recipe_errors_name_the_key(raw, word):
    with pytest.raises(ConfigError, match=word):
        Recipe.from_dict(raw)


def test_plan_mode_prints_and_runs_nothing(capsys):
    assert cli.main(["tiny-qwen2"]) == 0
    out = capsys.readouterr().out
    assert "tiny-qwen2" in out and "nothing executed" in out and "2 layers" in out and "max_new 16" in out
    assert cli.main(["tiny-qwen2", "--max-new", "5", "--dtype", "fp32"]) == 0        # command line beats the recipe
    out = capsys.readouterr().out
    assert "max_new 5" in out and "float32" in out


def test_refusals(capsys):
    for argv, word in ((["tiny-qwen2", "--mode", "serve"], "serve"), (["tiny-qwen2", "--cpu"], "CPU"),
                       (["tiny-qwen2", "--placement", "um"], "host-memory"), (["tiny-qwen2", "--tp", "2"], "one GPU"),
                       (["no-such-recipe"], "not found"),
                       (["tiny-qwen2", "--mode", "run", "--model-dir", "/nonexistent/dir"], "weights not found")):
        with pytest.raises(SystemExit) as e:
            cli.main(argv)
        assert word in str(e.value)
    assert cli.main(["--version"]) == 0
    assert "sllm-b200" in capsys.readouterr().out


def test_run_mode_on_cpu_ops(cpu_ops, capsys, monkeypatch):
    """--mode run with --random-weights, end to end with the CPU stand-in kernels."""
    import sllm_b200.engine.llm as llm_mod
    real = llm_mod.LLM

    def on_cpu(model_dir, **kw):
        kw.update(device="cpu", num_pages=32)
        return real(model_dir, **kw)
    monkeypatch.setattr(llm_mod, "LLM", on_cpu)
    assert cli.main(["tiny-qwen2", "--mode", "run", "--random-weights", "3", "--prompt-ids", "5,6,7", "--max-new", "4",
                     "--dtype", "float32", "--log-level", "ERROR"]) == 0
    ids = capsys.readouterr().out.strip().split(",")
    assert len(ids) == 4 and all(0 <= int(i) < 256 for i in ids)
    # several prompts at once, with the filters and the penalty of the sampler
    assert cli.main(["tiny-qwen2", "--mode", "run", "--random-weights", "3", "--batch", "one two", "three", "--max-new", "3",
                     "--temperature", "0.8", "--top-k", "5", "--top-p", "0.9", "--seed", "1", "--repetition-penalty", "1.2",
                     "--dtype", "float32", "--log-level", "ERROR"]) == 0
    out = capsys.readouterr().out.strip().splitlines()
    assert len(out) == 4 and out[0].startswith("['one two'] -> ") and out[2].startswith("['three'] -> ")
    assert len(out[0].split(" -> ")[1].split(",")) == 3
    assert cli.main(["tiny-qwen2", "--mode", "run", "--random-weights", "3", "--prompt", "abc", "--max-new", "2",
                     "--dtype", "float32", "--log-level", "ERROR"]) == 0
    assert len(capsys.readouterr().out.strip().splitlines()) == 2               # ids, then text


@pytest.mark.gpu
def test_launcher_runs_on_the_gpu(tmp_path):
    """`./sllm <recipe> --mode run --random-weights SEED --prompt-ids ...` as a user runs it, in a process
    of its own on the GPU with the real kernels: the ids it prints are the plain implementation's greedy
    tokens for the folder the same seed writes."""
    import subprocess

    from tests.conftest import cuda_or_skip
    from tests.plain import qwen2_plain as plain
    from sllm_b200.weights import write_random_model
    cuda_or_skip()
    root = os.path.dirname(RECIPES)
    prompt = [5, 17, 3, 200, 42, 7, 99, 120, 8, 61, 33, 250, 1]
    r = subprocess.run([os.path.join(root, "sllm"), "tiny-qwen2", "--mode", "run", "--random-weights", "0", "--prompt-ids",
                        ",".join(map(str, prompt)), "--max-new", "8", "--dtype", "float32", "--log-level", "ERROR"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [int(t) for t in r.stdout.strip().splitlines()[-1].split(",")]
    folder = write_random_model(str(tmp_path / "again"), resolve_recipe("tiny-qwen2", RECIPES).config_json(), 0,
                                std=0.02, bias_std=0.1)
    cfg, w = plain.load_model(folder)
    assert got == plain.generate(prompt, 8, w, cfg)
