"""The random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

Matrices, tables and biases are drawn from N(0, 0.02), norm weights are 1, and the values
are rounded to bfloat16 before they are stored, so that the bfloat16 engine, the float32
engine and a plain implementation all read the same numbers. The reference has the same
tool for its own container (tools/checkpoint.py:125-166; scripts/hf/synthetic.ts:81-116).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable

import torch

from ..parts.base import ParamSpec
from .safetensors_io import write_safetensors

STD = 0.02


def random_tensors(specs: Iterable[ParamSpec], seed: int, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Draws every tensor on the CPU in the order of ``specs`` from one generator."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for spec in specs:
        if spec.integer:
            out[spec.name] = torch.zeros(spec.shape, dtype=torch.int32)
        elif spec.init == "ones":
            out[spec.name] = torch.ones(spec.shape, dtype=dtype)
        elif spec.init == "zeros":
            out[spec.name] = torch.zeros(spec.shape, dtype=dtype)
        elif spec.init == "normal":
            out[spec.name] = (torch.randn(spec.shape, generator=gen, dtype=torch.float32) * STD).to(dtype)
        else:
            raise ValueError(f"{spec.name}: unknown init {spec.init!r}")
    return out


def write_random_model(config, out_dir: str, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """``config`` is a configuration object of a registered architecture."""
    from ..engine.model import model_param_specs  # parts and registries live above weights

    os.makedirs(out_dir, exist_ok=True)
    specs = model_param_specs(config.model_spec())
    tensors = random_tensors(specs, seed, dtype)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      {"format": "pt", "seed": str(int(seed))})
    tmp = os.path.join(out_dir, "config.json.tmp")
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(config.to_json(), f, indent=2, sort_keys=True)
        f.write("\n")
    os.replace(tmp, os.path.join(out_dir, "config.json"))
    return out_dir
