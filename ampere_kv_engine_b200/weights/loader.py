"""Weights from safetensors, by tensor name.

The reference lets the checkpoint library build a model object and reads tensors off it by
attribute (ampere_kv/runner.py:33-36).  Here the model says which tensors it wants
(name, shape, kind); the files are checked against that list before anything is read, and one
error lists everything that is missing, unexpected or of the wrong shape.

Kept dtypes: matrices and biases in the compute dtype (bfloat16 for serving), norm weights in
float32 (an exact widening; a tensor stored in 32-bit stays 32-bit), integer tables in int32.
"""

from __future__ import annotations

import json
import os

import torch
from safetensors import safe_open

from ..parts.base import ParamSpec

_FLOAT_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64}
_INT_DTYPES = {"I32": torch.int32, "I64": torch.int64, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8}


class WeightError(ValueError):
    """The checkpoint does not match the model: lists missing, unexpected and misshapen tensors."""


def checkpoint_files(model_dir: str) -> list[str]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as handle:
            weight_map = json.load(handle).get("weight_map", {})
        files = sorted(set(weight_map.values()))
        return [os.path.join(model_dir, f) for f in files]
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors")) if os.path.isdir(model_dir) else []
    if not files:
        raise WeightError(f"{model_dir}: no model.safetensors (or *.safetensors) in the model folder")
    return [os.path.join(model_dir, f) for f in files]


def _stored_dtype(handle, name: str) -> str:
    return handle.get_slice(name).get_dtype()


def check_against(specs: dict[str, ParamSpec], found: dict[str, tuple[tuple[int, ...], str]], where: str) -> None:
    """Raise one :class:`WeightError` naming every problem, or return."""
    missing = sorted(n for n, s in specs.items() if not s.optional and n not in found)
    unexpected = sorted(n for n in found if n not in specs)
    wrong_shape = sorted((n, specs[n].shape, found[n][0]) for n in found
                         if n in specs and tuple(found[n][0]) != tuple(specs[n].shape))
    wrong_dtype = []
    for n, (shape, dtype) in found.items():
        if n not in specs:
            continue
        table = specs[n].kind == "table"
        if (table and dtype not in _INT_DTYPES) or (not table and dtype not in _FLOAT_DTYPES):
            wrong_dtype.append((n, dtype))
    if not (missing or unexpected or wrong_shape or wrong_dtype):
        return
    lines = [f"{where}: the checkpoint does not match the model"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong_shape:
        lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
            f"{n} is {list(got)}, expected {list(exp)}" for n, exp, got in wrong_shape))
    if wrong_dtype:
        lines.append(f"  wrong dtype ({len(wrong_dtype)}): " + ", ".join(f"{n} is {d}" for n, d in sorted(wrong_dtype)))
    raise WeightError("\n".join(lines))


def cast_for(spec: ParamSpec, tensor: torch.Tensor, compute_dtype: torch.dtype) -> torch.Tensor:
    if spec.kind == "table":
        return tensor.to(torch.int32)
    if spec.kind == "vector":
        return tensor.to(torch.float32)
    return tensor.to(compute_dtype)


def load_weights(model, model_dir: str) -> None:
    """Fill ``model`` (a DecoderModel) from the safetensors files of ``model_dir``."""
    specs = model.param_specs()
    files = checkpoint_files(model_dir)
    found: dict[str, tuple[tuple[int, ...], str]] = {}
    where: dict[str, str] = {}
    for path in files:
        with safe_open(path, framework="pt", device="cpu") as handle:
            for name in handle.keys():
                sl = handle.get_slice(name)
                found[name] = (tuple(sl.get_shape()), sl.get_dtype())
                where[name] = path
    check_against(specs, found, model_dir)
    tensors: dict[str, torch.Tensor] = {}
    for path in files:
        with safe_open(path, framework="pt", device="cpu") as handle:
            for name in handle.keys():
                if name in specs and where[name] == path:
                    tensors[name] = cast_for(specs[name], handle.get_tensor(name), model.dtype).to(model.device)
    model.load_tensors(tensors)
