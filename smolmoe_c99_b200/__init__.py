"""A small, whole model library with generation of its own for one NVIDIA B200:
configuration, weights, parts, cache, step function, generation loop, sampling and the
CUDA kernels (sm_100a) under them, for the Qwen2 decoder."""

__version__ = "0.1.0"
