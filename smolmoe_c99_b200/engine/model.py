"""The decoder put together from a ``ModelSpec``: embedding, the layers' blocks in the order
the spec lists them, final norm and output head (reference: src/model.c:664-690 for the
forward pass, src/model.c:654-662 for the head on the wanted rows only)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import ModelSpec
from ..parts import BLOCKS, NORMS, ParamSpec, Runtime, full_name


def model_param_specs(spec: ModelSpec) -> List[ParamSpec]:
    """Every tensor the model needs, by name and shape."""
    out = [ParamSpec("embedding", spec.embedding_name, (spec.vocab_size, spec.hidden_size))]
    for layer in spec.layers:
        out += BLOCKS.get(layer.block).param_specs(layer)
    out += NORMS.get(spec.final_norm.kind).param_specs(spec.final_norm, spec.final_norm_prefix)
    if spec.head_name is not None:
        out.append(ParamSpec("head", spec.head_name, (spec.vocab_size, spec.hidden_size)))
    names = [s.name for s in out]
    if len(set(names)) != len(names):
        dup = sorted({n for n in names if names.count(n) > 1})
        raise ValueError(f"the model names a tensor twice: {', '.join(dup)}")
    return out


def cache_needs(spec: ModelSpec) -> list:
    """What each run of ``spec.order`` needs from the cache (see ``SequenceCache``)."""
    needs: list = []
    last_run_of: Dict[int, int] = {}
    for run, index in enumerate(spec.order):
        layer = spec.layers[index]
        if layer.cache_from is not None:
            if layer.cache_from not in last_run_of:
                raise ValueError(f"layer {index} reads the cache of layer {layer.cache_from}, which has not run before it")
            needs.append(last_run_of[layer.cache_from])
        else:
            needs.append(BLOCKS.get(layer.block).cache_need(layer))
        last_run_of[index] = run
    return needs


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.blocks = [BLOCKS.get(layer.block)(layer, runtime) for layer in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, runtime)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.embedding = tensors[self.spec.embedding_name]
        for block in self.blocks:
            block.bind(tensors)
        norm_specs = type(self.final_norm).param_specs(self.spec.final_norm, self.spec.final_norm_prefix)
        self.final_norm.bind({s.key: tensors[s.name] for s in norm_specs})
        # a tied head is the same device buffer as the embedding (src/modelfile.c:25-34)
        self.head = self.embedding if self.spec.head_name is None else tensors[self.spec.head_name]

    def forward(self, step, cache, want_rows: Optional[torch.Tensor], status: Optional[torch.Tensor] = None):
        """Runs the step's tokens through every layer; returns float logits ``[wanted, vocab]``
        for the packed token indices in ``want_rows`` (int32), or None when none are wanted."""
        ops = self.runtime.ops
        ops.lap(None)
        residual = ops.embedding(self.embedding, step.tokens, status)
        ops.lap("embed")
        for run, index in enumerate(self.spec.order):
            self.blocks[index].forward(residual, step, cache.run_view(run))
        if want_rows is None or want_rows.numel() == 0:
            return None
        every_row = getattr(step, "wants_every_row", False)   # the wanted rows are 0..T-1 in order
        x = self.final_norm.forward(residual, None if every_row else want_rows, lazy=True)
        logits = ops.linear(x, self.head, None, out_dtype=torch.float32)
        ops.lap("logits")
        return logits

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once (a tied head counts once)."""
        seen, total = set(), 0
        tensors = [self.embedding if self.head is self.embedding else self.head]
        for block in self.blocks:
            for part in (block.mixer_norm, block.mixer, block.feed_forward_norm, block.feed_forward):
                tensors += [v for v in vars(part).values() if isinstance(v, torch.Tensor)]
        tensors += [v for v in vars(self.final_norm).values() if isinstance(v, torch.Tensor)]
        for t in tensors:
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total
