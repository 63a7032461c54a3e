"""A small, whole model library with generation of its own for one NVIDIA B200:
configuration, weights, parts, cache, step function, generation loop, sampling and the
CUDA kernels (sm_100a) under them, for the Qwen2 decoder."""

__version__ = "0.1.0"


def __getattr__(name):
    # the entry point is imported on first use, so that configuration and weights work
    # (and can be tested) on a machine without a GPU
    if name == "Model":
        from .engine.entry import Model
        return Model
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)
