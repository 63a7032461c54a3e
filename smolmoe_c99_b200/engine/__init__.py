"""The engine: model, step function, generation loop and entry points."""
from .batch import StepBatch, pack_step
from .model import DecoderModel, cache_needs, model_param_specs

__all__ = ["DecoderModel", "StepBatch", "cache_needs", "model_param_specs", "pack_step"]
