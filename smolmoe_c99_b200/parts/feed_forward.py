"""The gated feed-forward: down(up(x) * act(gate(x))), added to the residual; gate and up
are one product (reference: src/model.c:547-561; SiLU: src/vecmath.c:78-81)."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from .base import FEED_FORWARDS, ParamSpec, Part, Runtime, full_name


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(Part):
    takes_lazy_norm = True

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden_size"])
        self.intermediate = int(spec["intermediate_size"])
        from ..kernels.ops import ACTIVATIONS
        self.activation = spec.get("activation", "silu")
        if self.activation not in ACTIVATIONS:     # the kernels fold the activation into the product's epilogue
            raise ValueError(f"gated_mlp: activation {self.activation!r} is not one the kernels know "
                             f"({', '.join(sorted(ACTIVATIONS))})")
        self.w_gate_up = self.w_down = None

    @classmethod
    def param_specs(cls, spec: PartSpec, prefix: str) -> List[ParamSpec]:
        d, h = int(spec["hidden_size"]), int(spec["intermediate_size"])
        n = spec.names
        return [ParamSpec("gate", full_name(prefix, n["gate"]), (h, d)),
                ParamSpec("up", full_name(prefix, n["up"]), (h, d)),
                ParamSpec("down", full_name(prefix, n["down"]), (d, h))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([tensors["gate"], tensors["up"]], dim=0).contiguous()
        self.w_down = tensors["down"]

    def forward(self, x: torch.Tensor, residual: torch.Tensor, step) -> None:
        ops = self.runtime.ops
        h = ops.gated_linear(x, self.w_gate_up, self.intermediate, self.runtime.dtype, self.activation)
        ops.lap("ffn_up")   # with the norm before it where that is the product's prologue, and the activation
        ops.linear(h, self.w_down, None, out=residual, accumulate=True)
        ops.lap("ffn_down")

    def fused_decode_record(self):
        """What a kernel that runs whole layers needs of this part; None for a subclass with a forward pass of its
        own, which is not what that kernel computes."""
        if type(self).forward is not GatedMLP.forward:
            return None
        if self.activation != "silu":
            return None
        return {"w_gate_up": self.w_gate_up, "w_down": self.w_down, "hidden": self.hidden, "intermediate": self.intermediate}
