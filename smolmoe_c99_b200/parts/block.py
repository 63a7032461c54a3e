"""Arrangements of a layer's parts. ``pre_norm``: x += mixer(norm(x)); x += ffn(norm(x))
(reference: src/model.c:504,631,683-686)."""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import LayerSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, ParamSpec, Runtime, full_name


@BLOCKS.register("pre_norm")
class PreNormBlock:
    def __init__(self, spec: LayerSpec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, runtime)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, runtime)
        self.feed_forward_norm = NORMS.get(spec.feed_forward_norm.kind)(spec.feed_forward_norm, runtime)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, runtime)

    @classmethod
    def parts(cls, spec: LayerSpec):
        """(registry, part spec) of every part, in the order their weights are listed."""
        return [(NORMS, spec.mixer_norm), (MIXERS, spec.mixer), (NORMS, spec.feed_forward_norm),
                (FEED_FORWARDS, spec.feed_forward)]

    @classmethod
    def param_specs(cls, spec: LayerSpec) -> List[ParamSpec]:
        out: List[ParamSpec] = []
        for registry, part in cls.parts(spec):
            out += registry.get(part.kind).param_specs(part, spec.weight_prefix)
        return out

    def bind(self, tensors) -> None:
        """``tensors``: full tensor name -> tensor."""
        for part in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward):
            specs = type(part).param_specs(part.spec, self.spec.weight_prefix)
            part.bind({s.key: tensors[s.name] for s in specs})

    @classmethod
    def cache_need(cls, spec: LayerSpec):
        mixer = MIXERS.get(spec.mixer.kind)
        return mixer.cache_need(spec.mixer) if hasattr(mixer, "cache_need") else None

    def forward(self, residual: torch.Tensor, step, cache) -> None:
        # a part that sets ``takes_lazy_norm`` hands its input straight to the kernel library's
        # products and may receive the norm as a handle; any other part gets a tensor
        ops = self.runtime.ops
        lazy = getattr(self.mixer, "takes_lazy_norm", False)
        x = self.mixer_norm.forward(residual, lazy=lazy)
        ops.lap("norm")
        self.mixer.forward(x, residual, step, cache)
        lazy = getattr(self.feed_forward, "takes_lazy_norm", False)
        x = self.feed_forward_norm.forward(residual, lazy=lazy)
        ops.lap("norm")
        self.feed_forward.forward(x, residual, step)

    def fused_decode_record(self, cache):
        """This layer as the fused decode step takes it (see ``Ops.decode_fused``), or None if one of its parts has
        no such description: x += mixer(norm(x)); x += ffn(norm(x)) with the parts' own records."""
        parts = (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
        if type(self).forward is not PreNormBlock.forward or not all(hasattr(part, "fused_decode_record") for part in parts):
            return None
        record = {"norm1": self.mixer_norm.fused_decode_record(), "mixer": self.mixer.fused_decode_record(cache),
                  "norm2": self.feed_forward_norm.fused_decode_record(), "ffn": self.feed_forward.fused_decode_record()}
        return None if any(v is None for v in record.values()) else record
