"""Shared fixtures: the tiny configurations, model folders in temporary
directories, and the CPU stand-in for the kernels."""

from __future__ import annotations

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


# The two tiny configurations differ in every size and option.
TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "max_position_embeddings": 128, "tie_word_embeddings": True,
    "hidden_act": "silu",
}
TINY_A_INIT = dict(seed=0, std=0.05, gain_std=0.1)
TINY_A_PAGE = 16

TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 320, "vocab_size": 384, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "max_position_embeddings": 256, "tie_word_embeddings": False,
    "hidden_act": "silu",
}
TINY_B_INIT = dict(seed=1, std=0.04, gain_std=0.1)
TINY_B_PAGE = 8

TINY = {"A": (TINY_A, TINY_A_INIT, TINY_A_PAGE), "B": (TINY_B, TINY_B_INIT, TINY_B_PAGE)}


def make_model_dir(tmp_path, config, init, storage="bfloat16", **over):
    from sllm_b200.weights import write_random_model
    cfg = dict(config)
    cfg.update(over)
    d = os.path.join(str(tmp_path), "model")
    # biases large enough that a wrong bias index shows (the reference's fixture
    # does the same, serving/dev_model.py:171-177)
    return write_random_model(d, cfg, init["seed"], std=init["std"], bias_std=6 * init["std"],
                              gain_std=init["gain_std"], storage=storage)


@pytest.fixture(params=["A", "B"])
def tiny(request, tmp_path):
    """(name, model folder, page size) for each tiny configuration."""
    config, init, page = TINY[request.param]
    return request.param, make_model_dir(tmp_path, config, init), page


@pytest.fixture
def cpu_ops(monkeypatch):
    """Put the PyTorch statements of the operations in the kernels' place, so that
    engine logic can run without a GPU.  Tests only."""
    import sllm_b200.ops as ops
    from tests import torch_ops
    for name in torch_ops.ALL:
        monkeypatch.setattr(ops, name, getattr(torch_ops, name))
    return ops


def cuda_or_skip():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return "cuda:0"
