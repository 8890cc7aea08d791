"""Random weights from a configuration and a seed.

Two uses: a model folder on disk (config.json + model.safetensors) that goes through the same
loader as a real checkpoint, and direct initialisation on the device for large benchmark
shapes.  Draws: matrices and biases N(0, 0.02), norm weights 1 + N(0, 0.1), one tensor after
the other in the model's declaration order from one seeded generator.  The reference has no
such mode (it needs the published checkpoint, ampere_kv/runner.py:13-14).
"""

from __future__ import annotations

import json
import os

import torch
from safetensors.torch import save_file

from ..parts.base import ParamSpec
from .loader import cast_for


def _draw(spec: ParamSpec, generator: torch.Generator, device) -> torch.Tensor:
    if spec.kind == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    noise = torch.randn(spec.shape, generator=generator, dtype=torch.float32, device=device)
    if spec.init == "norm":
        return 1.0 + 0.1 * noise
    if spec.init == "zeros":
        return torch.zeros_like(noise)
    return 0.02 * noise


def random_tensors(specs: dict[str, ParamSpec], seed: int, device="cpu") -> dict[str, torch.Tensor]:
    """float32 draws for every non-optional tensor, in declaration order."""
    generator = torch.Generator(device=device).manual_seed(seed)
    return {name: _draw(spec, generator, device) for name, spec in specs.items() if not spec.optional}


def init_random(model, seed: int) -> None:
    """Fill ``model`` in place with random weights drawn on its own device."""
    specs = model.param_specs()
    generator = torch.Generator(device=model.device).manual_seed(seed)
    tensors = {}
    for name, spec in specs.items():
        if spec.optional:
            continue
        tensors[name] = cast_for(spec, _draw(spec, generator, model.device), model.dtype)
    model.load_tensors(tensors)


def write_random_model(config, seed: int, out_dir: str, dtype: torch.dtype = torch.float32) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed configuration of a registered
    architecture); returns ``out_dir``.  ``dtype`` is the stored dtype of every tensor."""
    from ..models.decoder import DecoderModel
    from ..models.registry import ARCHITECTURES

    arch = ARCHITECTURES[config.architectures[0]]
    model = DecoderModel(arch.build_spec(config), dtype=torch.float32, device="cpu")
    tensors = {name: t.to(dtype).contiguous() for name, t in random_tensors(model.param_specs(), seed).items()}
    os.makedirs(out_dir, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.float16: "float16"}[dtype]
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(raw, handle, indent=2)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
    return out_dir
