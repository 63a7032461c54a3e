"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a :class:`~smolmoe_c99_b200.config.spec.PartSpec` (its sizes and
constants) and a :class:`Runtime` (dtype, device, kernels). No part knows which model it
is in. The reference has one fixed ``attention_block`` / ``ffn_block`` pair whose variants
are optional pointers in ``struct Layer`` (src/model.c:493-542,625-650); here each variant
is a class found by name.

Interfaces
----------
* every part: ``param_specs(spec, prefix)`` lists its tensors (name, shape, how random
  weights are drawn); ``bind(tensors)`` receives them by the part's own keys.
* norm: ``forward(residual) -> x`` -- fp32 rows in, rows of the compute dtype out.
* mixer: ``cache_need(spec)`` says what it keeps per sequence (keys and values of all or of
  a window of positions, a state of fixed size, or nothing);
  ``forward(x, residual, step, cache)`` adds its output to ``residual`` in place.
* feed-forward: ``forward(x, residual, step)`` adds its output to ``residual`` in place.
* position encoding: ``tables(max_positions, device)`` returns what the mixer's kernels
  index by absolute position.
* block: ``forward(residual, step, cache)`` runs the layer's parts in its arrangement.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Mapping, Optional, Tuple

import torch

from ..config.spec import PartSpec


@dataclass(frozen=True)
class ParamSpec:
    """One tensor of a part. ``init`` is how the random-weights mode draws it:
    ``normal`` (N(0, 0.02)), ``ones`` or ``zeros``. ``integer`` tables are kept as int32."""

    key: str
    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    integer: bool = False


@dataclass(frozen=True)
class KVNeed:
    """Keys and values per position: of every position (``window=None``) or of the last
    ``window`` positions."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A state of fixed size per sequence, zeroed when the sequence starts."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """What every part is built with: the compute dtype (bfloat16, or float32 for the true
    32-bit path), the device, and the kernel library."""

    dtype: torch.dtype
    device: torch.device
    ops: Any
    max_positions: int = 0


class Part:
    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime

    @classmethod
    def param_specs(cls, spec: PartSpec, prefix: str) -> List[ParamSpec]:
        return []

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        pass


def full_name(prefix: str, leaf: str) -> str:
    return f"{prefix}.{leaf}" if prefix else leaf


class Registry:
    """Name -> class for one kind of part."""

    def __init__(self, what: str):
        self.what = what
        self._classes: Dict[str, type] = {}

    def register(self, kind: str, cls: type = None):
        if cls is None:  # used as a decorator
            def deco(c):
                self._classes[kind] = c
                return c
            return deco
        self._classes[kind] = cls
        return cls

    def get(self, kind: str) -> type:
        if kind not in self._classes:
            known = ", ".join(sorted(self._classes)) or "none"
            raise KeyError(f"unknown {self.what} kind: {kind} (known: {known})")
        return self._classes[kind]

    def kinds(self) -> List[str]:
        return sorted(self._classes)


NORMS = Registry("norm")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block")
