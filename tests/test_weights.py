"""Loading by tensor name: dtypes kept, one error that lists everything wrong, the random-weights folder."""

import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import tiny
from ampere_kv_engine_b200.models.decoder import DecoderModel
from ampere_kv_engine_b200.models.registry import config_from_dict
from ampere_kv_engine_b200.weights.loader import WeightError, load_weights
from ampere_kv_engine_b200.weights.random_init import write_random_model
from plain import qwen3_plain as plain


def build(name, dtype=torch.float32):
    arch, cfg = config_from_dict(tiny.config(name))
    return cfg, DecoderModel(arch.build_spec(cfg), dtype=dtype, device="cpu")


def test_random_folder_round_trip_and_names(tmp_path):
    cfg, model = build("B")
    folder = write_random_model(cfg, 3, str(tmp_path / "m"), torch.float32)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    stored = load_file(os.path.join(folder, "model.safetensors"))
    # the names are the checkpoint's own: the plain implementation reads the same file by the same names
    assert set(stored) == set(plain.random_weights(tiny.config("B"), 0))
    load_weights(model, folder)
    attn = model.blocks[1].mixer
    want = torch.cat([stored[f"model.layers.1.self_attn.{p}_proj.weight"] for p in "qkv"])
    torch.testing.assert_close(attn.w_qkv, want, atol=0, rtol=0)
    assert attn.b_qkv is not None and attn.window == 40
    # same seed, same tensors; another seed, other tensors
    again = load_file(os.path.join(write_random_model(cfg, 3, str(tmp_path / "n"), torch.float32), "model.safetensors"))
    assert all(torch.equal(stored[k], again[k]) for k in stored)
    other = load_file(os.path.join(write_random_model(cfg, 4, str(tmp_path / "o"), torch.float32), "model.safetensors"))
    assert not torch.equal(stored["model.norm.weight"], other["model.norm.weight"])
    raw = json.load(open(os.path.join(folder, "config.json")))
    assert raw["architectures"] == ["Qwen3ForCausalLM"] and raw["sliding_window"] == 40


def test_tied_head_reads_the_embedding(tmp_path):
    cfg, model = build("A")
    folder = write_random_model(cfg, 1, str(tmp_path / "m"))
    assert "lm_head.weight" not in load_file(os.path.join(folder, "model.safetensors"))
    load_weights(model, folder)
    assert model.head.weight is model.embedding.weight


def test_kept_dtypes(tmp_path):
    """bfloat16 serving keeps matrices in bfloat16; norm weights are float32 whatever the file stores
    (a 32-bit tensor stays 32-bit, a 16-bit one is widened exactly)."""
    for stored in (torch.float32, torch.bfloat16):
        cfg, model = build("A", torch.bfloat16)
        folder = write_random_model(cfg, 1, str(tmp_path / f"m{stored}"), stored)
        load_weights(model, folder)
        assert model.embedding.weight.dtype == torch.bfloat16
        assert model.blocks[0].mixer.w_qkv.dtype == torch.bfloat16
        assert model.final_norm.weight.dtype == torch.float32
        assert model.blocks[0].mixer.q_norm_weight.dtype == torch.float32
        raw = load_file(os.path.join(folder, "model.safetensors"))["model.norm.weight"]
        torch.testing.assert_close(model.final_norm.weight, raw.float(), atol=0, rtol=0)
    cfg, model = build("A", torch.float32)
    load_weights(model, write_random_model(cfg, 1, str(tmp_path / "f"), torch.bfloat16))
    assert model.embedding.weight.dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    cfg, model = build("A")
    folder = write_random_model(cfg, 1, str(tmp_path / "m"))
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.ones(32)
    tensors["model.embed_tokens.weight"] = torch.zeros(512, 64, dtype=torch.int32)
    save_file(tensors, path)
    with pytest.raises(WeightError) as err:
        load_weights(model, folder)
    text = str(err.value)
    assert "missing (2): model.layers.1.mlp.up_proj.weight, model.norm.weight" in text
    assert "unexpected (1): model.layers.0.self_attn.rotary.inv_freq" in text
    assert "model.layers.0.self_attn.q_norm.weight is [32], expected [16]" in text
    assert "wrong dtype (1): model.embed_tokens.weight is I32" in text
    assert not model.loaded


def test_sharded_checkpoint_and_missing_files(tmp_path):
    cfg, model = build("A")
    folder = write_random_model(cfg, 1, str(tmp_path / "m"))
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    names = sorted(tensors)
    parts = {"model-00001-of-00002.safetensors": names[::2], "model-00002-of-00002.safetensors": names[1::2]}
    for fname, keys in parts.items():
        save_file({k: tensors[k] for k in keys}, os.path.join(folder, fname))
    os.remove(os.path.join(folder, "model.safetensors"))
    index = {"weight_map": {k: f for f, keys in parts.items() for k in keys}}
    json.dump(index, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    load_weights(model, folder)
    torch.testing.assert_close(model.final_norm.weight, tensors["model.norm.weight"], atol=0, rtol=0)
    with pytest.raises(WeightError, match="no model.safetensors"):
        load_weights(model, str(tmp_path))


def test_a_model_without_weights_cannot_run():
    from ampere_kv_engine_b200.engine.step import ModelRunner
    _, model = build("A")
    with pytest.raises(ValueError, match="no weights"):
        ModelRunner(model, num_pages=4)
