"""Tiny random model folders for the tests (made in a temporary folder, never committed) and the
plain implementation's logits for them."""

from __future__ import annotations

import functools
import os
import tempfile

import torch
from safetensors.torch import load_file

import tiny
from plain import qwen3_plain as plain


@functools.lru_cache(maxsize=None)
def model_folder(name: str, seed: int = 1, stored: str = "float32") -> str:
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.random_init import write_random_model
    _, cfg = config_from_dict(tiny.config(name))
    out = tempfile.mkdtemp(prefix=f"tiny_{name}_")
    write_random_model(cfg, seed, out, {"float32": torch.float32, "bfloat16": torch.bfloat16}[stored])
    return out


def plain_weights(folder: str, dtype: str) -> dict:
    """Checkpoint tensors as float32; for the bfloat16 comparison they are first rounded to bfloat16, so the
    plain model sees the values the engine computes with."""
    w = load_file(os.path.join(folder, "model.safetensors"))
    if dtype == "bfloat16":
        return {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    return {k: v.float() for k, v in w.items()}


def plain_logits(folder: str, raw_config: dict, requests: dict[str, list[int]], dtype: str) -> dict[str, torch.Tensor]:
    w = plain_weights(folder, dtype)
    return {rid: plain.forward_logits(w, raw_config, toks) for rid, toks in requests.items()}
