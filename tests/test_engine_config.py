"""The engine's options as one typed object: every refusal in one place, the context limit wired to the model's
positions and to submit, end-of-sequence ids from generation_config.json, a tied head that carries a tensor."""

import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import tiny
from ampere_kv_engine_b200.config.engine_config import EngineConfig, EngineConfigError
from ampere_kv_engine_b200.models.registry import config_from_dict, load_config
from ampere_kv_engine_b200.weights.loader import WeightError
from ampere_kv_engine_b200.weights.random_init import write_random_model


@pytest.mark.parametrize("bad", [
    dict(page_size=0), dict(page_size=True), dict(num_pages=-1), dict(max_seqs=0), dict(max_batch_tokens=0),
    dict(max_context=0), dict(max_tokens=1.5), dict(admission="greedy"), dict(dtype="float16"),
    dict(dtype="bfloat16", kv_dtype="float32"), dict(cuda_graphs=1), dict(lookahead="yes"),
])
def test_every_bad_option_is_refused_by_name(bad):
    with pytest.raises(EngineConfigError) as err:
        EngineConfig(**bad)
    assert any(name in str(err.value) for name in bad)


def test_names_defaults_and_derived_values():
    cfg = EngineConfig(dtype="fp32", kv_dtype=torch.float32, page_size=32, max_tokens=1000, max_seqs=5)
    assert cfg.dtype == "float32" and cfg.kv_dtype == "float32"
    done = cfg.resolved(max_position=512)
    assert done.max_context == 512 and done.num_pages == (1000 + 31) // 32 + 5
    assert EngineConfig(num_pages=7).resolved(100).num_pages == 7
    assert EngineConfig(max_context=64).resolved(100).max_context == 64
    with pytest.raises(EngineConfigError, match="max_context"):
        EngineConfig(max_context=101).resolved(100)
    with pytest.raises(EngineConfigError, match="unknown engine option"):
        cfg.replace(pagesize=16)


def _engine(fake_ext, name="A", **options):
    from ampere_kv_engine_b200.engine.engine import Engine
    from models_util import model_folder
    return Engine.from_pretrained(model_folder(name), device="cpu", config=EngineConfig(dtype="float32", **options))


def test_submit_refuses_more_than_the_models_positions(fake_ext):
    engine = _engine(fake_ext, num_pages=64)
    limit = tiny.config("A")["max_position_embeddings"]
    assert engine.config.max_context == limit
    scheduler = engine.new_scheduler()
    scheduler.submit("fits", [1] * (limit - 8), 8)
    with pytest.raises(ValueError, match="maximum context"):
        scheduler.submit("too long", [1] * (limit - 8), 9)
    with pytest.raises(ValueError, match="maximum context"):
        engine.generate([[1] * limit], max_new_tokens=1)
    # a narrower limit of the engine's own
    narrow = _engine(fake_ext, num_pages=64, max_context=40)
    with pytest.raises(ValueError, match="maximum context of 40"):
        narrow.generate([[1] * 33], max_new_tokens=8)
    assert narrow.generate([[1] * 32], max_new_tokens=8, ignore_eos=True)[0].__len__() == 8


def test_engine_refuses_a_dtype_that_is_not_the_models(fake_ext):
    from ampere_kv_engine_b200.engine.engine import Engine
    engine = _engine(fake_ext, num_pages=16)
    with pytest.raises(ValueError, match="dtype"):
        Engine(engine.model, EngineConfig(dtype="bfloat16"))
    assert Engine(engine.model, num_pages=16).config.dtype == "float32"     # no word on the dtype: the model's


def _folder_with(tmp_path, name, config_eos, generation_eos):
    _, cfg = config_from_dict(tiny.config(name))
    folder = write_random_model(cfg, 1, str(tmp_path / "m"))
    raw = json.load(open(os.path.join(folder, "config.json")))
    raw["eos_token_id"] = config_eos
    json.dump(raw, open(os.path.join(folder, "config.json"), "w"))
    if generation_eos is not None:
        json.dump({"eos_token_id": generation_eos}, open(os.path.join(folder, "generation_config.json"), "w"))
    return folder


def test_eos_ids_come_from_generation_config_when_it_has_them(tmp_path):
    """The reference stops on generation_config's ids (ampere_kv/runner.py:331); a published checkpoint lists an
    id there that its config.json does not."""
    folder = _folder_with(tmp_path, "A", 7, [7, 3])
    assert load_config(folder)[1].eos_token_id == (7, 3)
    json.dump({"do_sample": True}, open(os.path.join(folder, "generation_config.json"), "w"))
    assert load_config(folder)[1].eos_token_id == (7,)
    os.remove(os.path.join(folder, "generation_config.json"))
    assert load_config(folder)[1].eos_token_id == (7,)


def test_generation_stops_on_an_id_only_generation_config_names(fake_ext, tmp_path):
    from ampere_kv_engine_b200.engine.engine import Engine
    folder = _folder_with(tmp_path, "A", None, None)
    options = EngineConfig(dtype="float32", num_pages=32)
    prompt = [5, 9, 300, 41, 77]
    free = Engine.from_pretrained(folder, device="cpu", config=options).generate([prompt], max_new_tokens=12)[0]
    assert len(free) == 12
    stop = free[4]
    first = free.index(stop)
    folder = _folder_with(tmp_path, "A", 511 if stop != 511 else 510, [stop])
    got = Engine.from_pretrained(folder, device="cpu", config=options).generate([prompt], max_new_tokens=12)[0]
    assert got == free[:first + 1]


def test_tied_checkpoint_that_carries_a_head(tmp_path):
    """Equal to the embedding: accepted.  Different: one clear error, not silence."""
    from ampere_kv_engine_b200.models.decoder import DecoderModel
    from ampere_kv_engine_b200.weights.loader import load_weights
    arch, cfg = config_from_dict(tiny.config("A"))
    assert cfg.tie_word_embeddings
    folder = write_random_model(cfg, 1, str(tmp_path / "m"))
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, path)
    model = DecoderModel(arch.build_spec(cfg), dtype=torch.float32, device="cpu")
    load_weights(model, folder)
    assert model.head.weight is model.embedding.weight
    tensors["lm_head.weight"][3, 5] += 0.25
    save_file(tensors, path)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(DecoderModel(arch.build_spec(cfg), dtype=torch.float32, device="cpu"), folder)
