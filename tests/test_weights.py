"""The loader: round trip, dtypes kept, one error that lists every fault."""

import json
import os
import struct

import pytest
import torch

from sllm_b200.engine import build_model
from sllm_b200.weights import (SafetensorsError, SafetensorsFile, TensorSource, WeightError, write_random_model,
                               write_safetensors)
from sllm_b200.weights.safetensors_io import parse_header
from tests.conftest import TINY_A, TINY_A_INIT, TINY_B, TINY_B_INIT, make_model_dir


def test_round_trip_keeps_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5).bfloat16(), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
         "d": torch.randn(2, 2).half()}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    f = SafetensorsFile(p)
    assert f.tensor("a").dtype == torch.bfloat16 and torch.equal(f.tensor("a"), t["a"])
    assert f.tensor("b").dtype == torch.float32 and torch.equal(f.tensor("b"), t["b"])
    assert f.tensor("c").dtype == torch.int32 and torch.equal(f.tensor("c").long(), t["c"])
    assert f.tensor("d").dtype == torch.float16
    # the stock reader of the format agrees with the writer
    from safetensors.torch import load_file
    other = load_file(p)
    assert all(torch.equal(other[k], t[k]) for k in t)


def test_corrupt_files(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    with open(p, "wb") as f:
        f.write(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="8-byte"):
        parse_header(p)
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40))
    with pytest.raises(SafetensorsError, match="plausible"):
        parse_header(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)           # truncated data
    with pytest.raises(SafetensorsError, match="past the end"):
        parse_header(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="needs 16"):
        parse_header(p)
    hdr = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        parse_header(p)


def test_random_model_is_reproducible_and_loads(tmp_path):
    a = make_model_dir(tmp_path / "1", TINY_A, TINY_A_INIT)
    b = make_model_dir(tmp_path / "2", TINY_A, TINY_A_INIT)
    sa, sb = TensorSource(a), TensorSource(b)
    assert sorted(sa.names()) == sorted(sb.names())
    assert all(torch.equal(sa.tensor(n), sb.tensor(n)) for n in sa.names())
    assert "lm_head.weight" not in sa.names()                      # tied
    assert sa.tensor("model.embed_tokens.weight").dtype == torch.bfloat16
    model, cfg = build_model(a, "float32", "cpu")
    assert model.head is model.embedding
    assert model.layers[0].mixer.qkv.weight.dtype == torch.float32
    assert model.layers[0].parts["mixer_norm"].weight.dtype == torch.float32
    c = make_model_dir(tmp_path / "3", TINY_B, TINY_B_INIT, storage="float32")
    sc = TensorSource(c)
    assert "lm_head.weight" in sc.names() and sc.tensor("lm_head.weight").dtype == torch.float32
    model, _ = build_model(c, "bfloat16", "cpu")
    assert model.head is not model.embedding and model.head.dtype == torch.bfloat16
    assert model.layers[0].mixer.qkv_b.dtype == torch.float32       # biases and gains stay 32-bit


def _rewrite(model_dir, fn):
    src = TensorSource(model_dir)
    t = {n: src.tensor(n).clone() for n in src.names()}
    fn(t)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), t)


def test_one_error_lists_everything(tmp_path):
    d = make_model_dir(tmp_path, TINY_B, TINY_B_INIT)

    def damage(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.extra.weight"] = torch.zeros(3)
        t["model.layers.2.self_attn.o_proj.weight"] = torch.zeros(5, 5)
        del t["model.layers.0.self_attn.k_proj.bias"]               # q/k/v biases come as a set
    _rewrite(d, damage)
    with pytest.raises(WeightError) as ei:
        build_model(d, "float32", "cpu")
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.extra.weight"]
    assert e.wrong_shape == [("model.layers.2.self_attn.o_proj.weight", (96, 96), (5, 5))]
    assert any("k_proj.bias" in o for o in e.other)
    msg = str(e)
    for word in ("up_proj", "model.norm.weight", "extra.weight", "expected (96, 96), found (5, 5)"):
        assert word in msg


def test_untied_model_needs_its_head_and_tied_ignores_a_copy(tmp_path):
    d = make_model_dir(tmp_path / "u", TINY_B, TINY_B_INIT)
    _rewrite(d, lambda t: t.pop("lm_head.weight"))
    with pytest.raises(WeightError, match="lm_head.weight"):
        build_model(d, "float32", "cpu")
    d = make_model_dir(tmp_path / "t", TINY_A, TINY_A_INIT)
    _rewrite(d, lambda t: t.__setitem__("lm_head.weight", torch.zeros(256, 64)))
    with pytest.warns(UserWarning, match="lm_head.weight is in the checkpoint and not used"):
        model, _ = build_model(d, "float32", "cpu")
    assert model.head is model.embedding


def test_bias_free_checkpoint_loads(tmp_path):
    from sllm_b200.weights import write_random_model
    d = write_random_model(str(tmp_path / "nb"), dict(TINY_A), 3, include_optional=False)
    model, _ = build_model(d, "float32", "cpu")
    assert model.layers[0].mixer.qkv_b is None


def test_missing_folder_and_shards(tmp_path):
    with pytest.raises(WeightError, match="no .*safetensors"):
        TensorSource(str(tmp_path))
    d = make_model_dir(tmp_path, TINY_A, TINY_A_INIT)
    src = TensorSource(d)
    names = src.names()
    half = len(names) // 2
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), {n: src.tensor(n).clone() for n in names[:half]})
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), {n: src.tensor(n).clone() for n in names[half:]})
    wm = {n: "model-00001-of-00002.safetensors" for n in names[:half]}
    wm.update({n: "model-00002-of-00002.safetensors" for n in names[half:]})
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": wm}, f)
    os.remove(os.path.join(d, "model.safetensors"))
    model, _ = build_model(d, "float32", "cpu")
    assert model.embedding.shape == (256, 64)


def test_upload_is_refused_when_the_device_has_no_room(monkeypatch):
    """The guard before the upload: the bytes come from the tensor specs, the free bytes from the device
    (a fake here); too little room is a MemoryError that says how much is needed and how much is free."""
    import torch
    from sllm_b200.engine import loading
    from sllm_b200.config.registry import architecture_of
    from sllm_b200.models.causal_lm import CausalLM
    cfg = dict(TINY_A)
    arch = architecture_of(cfg)
    model = CausalLM(arch.plan(arch.config_cls.from_dict(cfg)), dtype=torch.bfloat16, device="cpu")
    need = loading.resident_bytes(model)
    specs = model.tensor_specs()
    by_hand = sum(int(torch.tensor(s.shape).prod()) * (4 if s.role in ("gain", "bias") else 2) for s in specs)
    assert need == by_hand and need > 0
    loading.check_device_memory(model)                      # a CPU model: nothing to check
    model.device = torch.device("cuda:0")
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda dev=None: (need + loading.SLACK_BYTES - 1, 10 * need))
    with pytest.raises(MemoryError) as e:
        loading.check_device_memory(model)
    assert "GiB" in str(e.value) and "free" in str(e.value)
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda dev=None: (need + loading.SLACK_BYTES, 10 * need))
    loading.check_device_memory(model)
