"""The parts a layer is put together from: norm, position encoding, mixer, feed-forward,
and their arrangement in a block; each found by name in a registry."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, KVNeed, ParamSpec, Part, Registry, Runtime,
                   StateNeed, full_name)
from . import norm, position, attention, feed_forward, block  # noqa: F401  (they register themselves)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "KVNeed", "ParamSpec", "Part", "Registry",
           "Runtime", "StateNeed", "full_name"]
