"""Rotary position encoding: tables of cos and sin by absolute position.

inv_freq_i = theta^(-2i/R) and angle = position * inv_freq_i are computed in double, cos
and sin are rounded to float (reference: src/model.c:166-169,425-437). The rotation itself
happens in the mixer's kernel on pairs (i, i + R/2): the reference rotates adjacent pairs
of weights that its converter permuted from this order (scripts/hf/permute.ts:14-28), which
is the same function of the unpermuted weights.
"""
from __future__ import annotations

from typing import Tuple

import torch

from ..config.spec import PartSpec
from .base import POSITIONS, ParamSpec, Part, Runtime, full_name


@POSITIONS.register("rope")
class RotaryPosition(Part):
    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec["rotary_dim"])
        if self.rotary_dim % 2:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even")
        self._tables = None

    def tables(self, n_positions: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """``(cos, sin)``, each float ``[n_positions, rotary_dim / 2]`` on the device."""
        if self._tables is None or self._tables[0].shape[0] < n_positions:
            half = self.rotary_dim // 2
            i = torch.arange(half, dtype=torch.float64)
            inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -(2.0 * i) / self.rotary_dim)
            angle = torch.arange(n_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
            self._tables = (torch.cos(angle).float().to(self.runtime.device).contiguous(),
                            torch.sin(angle).float().to(self.runtime.device).contiguous())
        return self._tables


@POSITIONS.register("none")
class NoPosition(Part):
    """Leaves q and k as they are (a rotation by zero)."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.rotary_dim = 0
        self._tables = None

    def tables(self, n_positions: int):
        if self._tables is None or self._tables[0].shape[0] < n_positions:
            z = torch.zeros((n_positions, 0), dtype=torch.float32, device=self.runtime.device)
            self._tables = (z, z.clone())
        return self._tables


@POSITIONS.register("learned")
class LearnedPositions(Part):
    """A table of position vectors that is added to the embeddings (an absolute position encoding): the kind of
    encoding that belongs to the model's first step, not to a mixer. ``add_to`` adds row ``position`` of the table to
    every token's row of the residual."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.size, self.positions = int(spec["size"]), int(spec["positions"])
        self.rotary_dim = 0
        self.table = None

    @classmethod
    def param_specs(cls, spec: PartSpec, prefix: str):
        return [ParamSpec("table", full_name(prefix, spec.names["table"]), (int(spec["positions"]), int(spec["size"])))]

    def bind(self, tensors) -> None:
        self.table = tensors["table"]

    def add_to(self, residual: torch.Tensor, step) -> None:
        self.runtime.ops.add_rows_(residual, self.table, step.positions)
