"""Binding weights by tensor name.

The model says which tensors it needs (name and shape); the folder says which it has.
Every disagreement -- missing, unexpected, wrong shape, wrong kind of number -- is
collected and reported in ONE error. The reference reports the first one only
("missing tensor: %s", "wrong tensor shape/type: %s", src/modelfile.c:117-135; "tensor
count does not match config", src/model.c:127-128; "unused source tensors",
scripts/hf/pipeline.ts:69-88).

Dtypes: floating-point tensors are kept in bfloat16 for the bfloat16 engine, except that
a tensor stored in 32-bit stays in 32-bit; the float32 engine widens everything to
float32 (exact). Integer tables become int32.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Sequence

import torch

from ..parts.base import ParamSpec
from .safetensors_io import SafetensorsError, open_checkpoint


class WeightsError(ValueError):
    """The folder's tensors do not match what the model needs."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str], wrong: Sequence[str]):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong = list(wrong)
        lines = [f"{where}: weights do not match the configuration"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shape or type ({len(self.wrong)}): " + "; ".join(self.wrong))
        super().__init__("\n".join(lines))


def stored_dtype(file_dtype: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    """The dtype a floating-point tensor is kept in on the device."""
    if engine_dtype == torch.float32:
        return torch.float32
    if file_dtype in (torch.float32, torch.float64):
        return torch.float32  # stored in 32-bit (or wider): stays 32-bit
    return torch.bfloat16


def load_weights(model_dir: str, specs: Iterable[ParamSpec], dtype: torch.dtype,
                 device: torch.device) -> Dict[str, torch.Tensor]:
    """Returns ``{tensor name: device tensor}`` for exactly the tensors in ``specs``."""
    specs = list(specs)
    try:
        available = open_checkpoint(model_dir)
    except SafetensorsError as e:
        raise WeightsError(str(e), [], [], []) from None
    wanted = {s.name: s for s in specs}
    missing = [n for n in wanted if n not in available]
    unexpected = sorted(n for n in available if n not in wanted)
    wrong: List[str] = []
    for name, spec in wanted.items():
        if name not in available:
            continue
        entry = available[name][1]
        if tuple(entry.shape) != tuple(spec.shape):
            wrong.append(f"{name}: expected {list(spec.shape)}, found {list(entry.shape)}")
        elif spec.integer == entry.dtype.is_floating_point or entry.dtype == torch.bool:
            kind = "an integer table" if spec.integer else "floating point"
            wrong.append(f"{name}: expected {kind}, found {entry.dtype}")
    if missing or unexpected or wrong:
        raise WeightsError(model_dir, missing, unexpected, wrong)
    out: Dict[str, torch.Tensor] = {}
    for name, spec in wanted.items():
        st, entry = available[name]
        host = st.tensor(name)
        target = torch.int32 if spec.integer else stored_dtype(entry.dtype, dtype)
        if not spec.integer and not bool(torch.isfinite(host.float()).all()):
            # the reference refuses non-finite weights at load (src/modelfile.c:137-185)
            raise WeightsError(model_dir, [], [], [f"{name}: holds a non-finite value"])
        out[name] = host.to(device=device, dtype=target, copy=True).contiguous()
    return out
