"""Architecture-neutral description of a decoder: what the engine builds from.

A configuration class (one per architecture) turns its own ``config.json`` keys into a
:class:`ModelSpec`. Everything below the configuration -- weights, parts, cache, step
function -- reads only the spec, so no part knows which model it is in.

The reference keeps the same information in one flat ``struct Config`` plus optional
pointers in ``struct Layer`` (src/config.h:13-27, src/model.h:25-30); here it is data per
layer so that layers of one model may differ.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: its kind (a registry key) and its sizes and constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    # the part's own tensors -> their names in the weight file, relative to the layer's
    # prefix (for the final norm: to ``ModelSpec.final_norm_prefix``)
    names: Mapping[str, str] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement of its parts and where its weights are found.

    ``cache_from`` names another layer (by index into ``ModelSpec.layers``) whose cache
    this layer's mixer reads instead of owning one; ``None`` means it owns its cache.
    """

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    weight_prefix: str
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder. ``order`` is the list of layer indices in the order they run;
    it may name a layer twice."""

    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding_name: str
    final_norm: PartSpec
    final_norm_prefix: str
    head_name: Optional[str]  # None: the head shares the embedding table (tied)
    layers: Tuple[LayerSpec, ...]
    order: Tuple[int, ...]
    stop_token_ids: Tuple[int, ...] = ()
    # steps of the model that belong to no layer; the defaults are "none of it" (the Qwen2 decoder has none:
    # embed_scale = 1 and plain logits, src/model.c:667,654-662 of the reference)
    embedding_scale: float = 1.0                      # the embeddings are multiplied by this
    embedding_position: Optional[PartSpec] = None     # a position encoding that is ADDED to the embeddings (kind "learned"), its
                                                      # tensors named relative to ``embedding_position_prefix``
    embedding_position_prefix: str = ""
    head_bias_name: Optional[str] = None              # a bias on the output head
    logit_softcap: Optional[float] = None             # logits = cap * tanh(logits / cap)

    def __post_init__(self) -> None:
        for index in self.order:
            if not 0 <= index < len(self.layers):
                raise ValueError(f"layer order names layer {index}, model has {len(self.layers)}")
        for number, layer in enumerate(self.layers):
            src = layer.cache_from
            if src is not None:
                if not 0 <= src < len(self.layers) or src == number:
                    raise ValueError(f"layer {number}: cache_from={src} is not another layer")
                if self.layers[src].cache_from is not None:
                    raise ValueError(f"layer {number}: cache_from={src} does not own a cache")


def require_keys(raw: Mapping[str, Any], keys: Sequence[str], where: str) -> None:
    """Every key must be present; the error names all that are missing."""
    missing = [k for k in keys if k not in raw or raw[k] is None]
    if missing:
        raise ConfigError(f"{where}: missing required key(s): {', '.join(missing)}")


class ConfigError(ValueError):
    """A configuration that cannot be used; the message names the key."""
