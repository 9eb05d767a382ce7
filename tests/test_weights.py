"""Weights: the container, loading by name, the one error that lists everything, random folders."""

import json
import os
import struct

import pytest
import torch

import helpers
from ferrisinfer_b200.errors import WeightFileError, WeightLoadError
from ferrisinfer_b200.weights import (SafetensorsFolder, check_tensors, inspect_folder, load_model, random_tensors,
                                      write_model_folder, write_safetensors)
from helpers import TINY_A, TINY_B


def test_container_round_trip_and_agreement_with_the_safetensors_package(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32)}
    path = tmp_path / "model.safetensors"
    write_safetensors(str(path), tensors)
    from safetensors.torch import load_file

    theirs = load_file(str(path))
    ours = SafetensorsFolder(str(tmp_path))
    assert sorted(ours.names()) == ["a", "b", "c"]
    for n, t in tensors.items():
        assert torch.equal(theirs[n], t) and torch.equal(ours.read(n), t) and ours.read(n).dtype == t.dtype


def test_sharded_folder(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), {"x": torch.ones(2, 2)})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"y": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    st = SafetensorsFolder(str(tmp_path))
    assert st.shape("x") == (2, 2) and torch.equal(st.read("y"), torch.zeros(3))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "gone.safetensors"}}))
    with pytest.raises(WeightFileError, match="gone.safetensors"):
        SafetensorsFolder(str(tmp_path))


def _raw(tmp_path, header: dict, data: bytes, name="model.safetensors"):
    text = json.dumps(header).encode()
    (tmp_path / name).write_bytes(struct.pack("<Q", len(text)) + text + data)


def test_malformed_files(tmp_path):
    with pytest.raises(WeightFileError, match="neither"):
        SafetensorsFolder(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(WeightFileError, match="truncated"):
        SafetensorsFolder(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(WeightFileError, match="beyond"):
        SafetensorsFolder(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", 4) + b"\xff\xfe\x00\x01")
    with pytest.raises(WeightFileError, match="JSON"):
        SafetensorsFolder(str(tmp_path))
    _raw(tmp_path, {"t": {"dtype": "F32", "shape": [2]}}, b"")
    with pytest.raises(WeightFileError, match="lacks"):
        SafetensorsFolder(str(tmp_path))
    _raw(tmp_path, {"t": {"dtype": "F32", "shape": [2], "data_offsets": [8, 0]}}, b"\0" * 8)
    with pytest.raises(WeightFileError, match="end < start"):
        SafetensorsFolder(str(tmp_path))
    _raw(tmp_path, {"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(WeightFileError, match="needs 12"):
        SafetensorsFolder(str(tmp_path))
    _raw(tmp_path, {"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8)
    with pytest.raises(WeightFileError, match="beyond the end"):
        SafetensorsFolder(str(tmp_path))
    _raw(tmp_path, {"t": {"dtype": "Q4_0", "shape": [4], "data_offsets": [0, 2]}}, b"\0" * 2)
    with pytest.raises(WeightFileError, match="Q4_0"):
        SafetensorsFolder(str(tmp_path))


def test_random_folder_is_seeded_and_fits(tmp_path):
    a = random_tensors(TINY_A, seed=5)
    b = random_tensors(TINY_A, seed=5)
    c = random_tensors(TINY_A, seed=6)
    assert all(torch.equal(a[n], b[n]) for n in a) and any(not torch.equal(a[n], c[n]) for n in a)
    assert "lm_head.weight" not in a and "lm_head.weight" in random_tensors(TINY_B, seed=5)
    w = a["model.layers.1.mlp.down_proj.weight"].float()
    assert a["model.layers.1.mlp.down_proj.weight"].dtype == torch.bfloat16 and abs(w.std().item() - 0.02) < 0.003
    n = a["model.norm.weight"].float()
    assert abs(n.mean().item() - 1.0) < 0.02
    folder = write_model_folder(TINY_B, 9, str(tmp_path / "m"), store_dtype="float32")
    report = inspect_folder(folder)
    assert report["problems"] is None and report["stored_dtypes"] == ["float32"]
    assert report["architecture"] == "Qwen2ForCausalLM"
    with open(os.path.join(folder, "config.json")) as f:
        assert json.load(f)["sliding_window"] == 21


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    tensors = random_tensors(TINY_A, seed=1)
    del tensors["model.layers.0.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    folder = tmp_path / "broken"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(str(folder / "model.safetensors"), tensors)
    with pytest.raises(WeightLoadError) as e:
        load_model(str(folder), "float32", "cpu")
    err = e.value
    assert err.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert err.wrong_shape == [("model.layers.1.self_attn.k_proj.weight", (32, 64), (16, 64))]
    text = str(err)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "expected [32, 64], found [16, 64]"):
        assert needle in text
    assert inspect_folder(str(folder))["problems"]["missing"] == err.missing


def test_biases_are_optional_and_a_tied_head_in_the_folder_is_ignored(tmp_path):
    from ferrisinfer_b200.config import resolve_config
    from ferrisinfer_b200.parts import build_model

    arch, cfg = resolve_config(TINY_A)
    specs = build_model(arch.plan(cfg)).tensor_specs()
    tensors = random_tensors(TINY_A, seed=1, optional=False)
    assert not any(n.endswith(".bias") for n in tensors)
    check_tensors(specs, {n: t.shape for n, t in tensors.items()})
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    check_tensors(specs, {n: t.shape for n, t in tensors.items()}, ignorable=("lm_head.weight",))
    with pytest.raises(WeightLoadError):
        check_tensors(specs, {n: t.shape for n, t in tensors.items()})


def test_dtypes_on_the_device_follow_the_roles(tmp_path):
    """bfloat16 matrices stay bfloat16; vectors are widened exactly; float32 mode widens everything."""
    folder = helpers.make_folder(tmp_path, TINY_A, seed=2)
    model, _ = load_model(folder, "bfloat16", "cpu")
    block = model.blocks[0]
    assert block.mixer.qkv_weight.dtype == torch.bfloat16 and block.mixer.qkv_weight.shape == (64 + 2 * 32, 64)
    assert block.mixer.qkv_bias.dtype == torch.float32 and block.mixer_norm.weight.dtype == torch.float32
    assert model.output.weight is model.embedding.weight  # tied
    _, stored = helpers.read_folder(folder)
    assert torch.equal(block.mixer_norm.weight, stored["model.layers.0.input_layernorm.weight"].float())
    assert torch.equal(block.mixer.qkv_weight[:64], stored["model.layers.0.self_attn.q_proj.weight"])
    model32, _ = load_model(folder, "float32", "cpu")
    assert model32.blocks[0].feed_forward.gate_up.dtype == torch.float32
    assert torch.equal(model32.blocks[0].feed_forward.gate_up[128:], stored["model.layers.0.mlp.up_proj.weight"].float())


def test_tensors_nobody_asks_for_are_an_error_unless_told_otherwise(tmp_path):
    """By default a tensor that no part asks for stands in the one error; with strict=False the folder loads and
    the model says which tensors it left alone.  Missing tensors and wrong shapes stay errors either way."""
    tensors = random_tensors(TINY_A, seed=4)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    folder = tmp_path / "extra"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(str(folder / "model.safetensors"), tensors)
    with pytest.raises(WeightLoadError):
        load_model(str(folder), "float32", "cpu")
    model, _ = load_model(str(folder), "float32", "cpu", strict=False)
    assert model.unexpected_tensors == ["model.layers.0.self_attn.rotary_emb.inv_freq"] and model.bound
    del tensors["model.norm.weight"]
    write_safetensors(str(folder / "model.safetensors"), tensors)
    with pytest.raises(WeightLoadError) as e:
        load_model(str(folder), "float32", "cpu", strict=False)
    assert e.value.missing == ["model.norm.weight"] and e.value.unexpected


@pytest.mark.gpu
def test_a_folder_goes_to_the_device_through_pinned_staging_buffers(tmp_path, monkeypatch):
    """Tensors larger than a staging buffer are sent in pieces, shards are read through their own mappings, and what
    arrives on the device is bit for bit what the safetensors package reads from the same files."""
    from ferrisinfer_b200.weights import loader

    monkeypatch.setattr(loader, "STAGING_BYTES", 4096)  # the embedding of 256 x 64 bf16 is 32 KB: eight pieces
    folder = helpers.make_folder(tmp_path, TINY_A, seed=6)
    _, stored = helpers.read_folder(folder)
    for dtype in ("bfloat16", "float32"):
        model, _ = load_model(folder, dtype, "cuda")
        want = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        assert model.embedding.weight.dtype == want and model.embedding.weight.is_cuda
        assert torch.equal(model.embedding.weight.cpu(), stored["model.embed_tokens.weight"].to(want))
        for l, block in enumerate(model.blocks):
            p = f"model.layers.{l}"
            assert torch.equal(block.feed_forward.down.cpu(), stored[f"{p}.mlp.down_proj.weight"].to(want))
            assert torch.equal(block.mixer.qkv_bias.cpu()[:64], stored[f"{p}.self_attn.q_proj.bias"].float())
            assert torch.equal(block.mixer_norm.weight.cpu(), stored[f"{p}.input_layernorm.weight"].float())
