"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * w, computed in float
(reference: src/model.c:334-342). The residual rows come in as float; the result has the
compute dtype of the engine."""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..config.spec import PartSpec
from .base import NORMS, ParamSpec, Part, Runtime, full_name


@NORMS.register("rmsnorm")
class RMSNorm(Part):
    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, spec: PartSpec, prefix: str) -> List[ParamSpec]:
        return [ParamSpec("weight", full_name(prefix, spec.names["weight"]), (int(spec["size"]),), init="ones")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def forward(self, residual: torch.Tensor, rows: Optional[torch.Tensor] = None, lazy: bool = False):
        """``rows`` (int32) picks which rows of ``residual`` are normalised. With ``lazy`` the
        result is a handle that the kernel library's products accept in place of a tensor (a
        product over a handful of tokens then computes the norm itself); ``.tensor()`` of the
        handle gives the values."""
        if lazy:
            return self.runtime.ops.rmsnorm_lazy(residual, self.weight, self.eps, self.runtime.dtype, rows)
        return self.runtime.ops.rmsnorm(residual, self.weight, self.eps, self.runtime.dtype, rows)

    def fused_decode_record(self):
        """What a kernel that runs whole layers needs of this part: ``(weight, eps)``; None for a subclass with a
        forward pass of its own, which is not what that kernel computes."""
        if type(self).forward is not RMSNorm.forward:
            return None
        return self.weight, self.eps
