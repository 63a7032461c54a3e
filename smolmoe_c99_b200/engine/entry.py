"""The Python entry point: open a model folder (or make random weights), generate.

The reference has no Python entry point; its C API is an opaque handle, an options struct
and a sink with callbacks (src/desktop.h:35-72, src/engine_sink.h:9-23). This follows that
shape and keeps the reference's names and meanings of options where it has them (``tokens``,
``temperature``, ``top_k``, ``top_p``, ``seed``, ``context``: src/main.c:98-110). ``batch`` is
the number of sequences that start together; in the reference it is a number of prompt
tokens per pass of its single sequence (src/main.c:106); its counterpart here is
``step_tokens``, the most tokens one step may bring.

    from smolmoe_c99_b200 import Model
    model = Model.from_folder("path/to/folder")            # config.json + model.safetensors
    out = model.generate([[1, 2, 3], [4, 5]], tokens=16)   # token ids in, token ids out
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence, Union

import torch

from ..sampling import Sampler, SamplingOptions
from .engine import Engine
from .generate import Completion, GenerationOptions, GenerationStats, TokenSink, generate

DEFAULT_CONTEXT = 2048   # src/main.c:746-747: min(the model's limit, 2048) unless --context is given


class Model:
    def __init__(self, engine: Engine):
        self.engine = engine
        self.last_stats: Optional[GenerationStats] = None

    # ---- opening -------------------------------------------------------------------------
    @classmethod
    def from_folder(cls, path: str, dtype: str = "bfloat16", context: Optional[int] = None, batch: int = 8,
                    device: str = "cuda:0", step_tokens: Optional[int] = None, kernels: str = "fast") -> "Model":
        """``context``: positions a sequence may hold (default: the smaller of the model's limit
        and 2048); ``batch``: most sequences that start together. The cache is sized for
        ``batch`` sequences of ``context`` positions. ``step_tokens``: the most tokens one step may bring; longer
        prompts go through in portions (the reference's ``--batch``, src/main.c:106). ``kernels``: ``"fast"`` or
        ``"plain"`` (every product and attention on the plain kernels, for comparison)."""
        from ..config import load_config

        limit = load_config(path).model_spec().max_positions
        context = min(limit, context or DEFAULT_CONTEXT)
        rounded = -(-context // 64) * 64
        return cls(Engine(path, dtype, max_tokens=rounded * batch, max_slots=batch, max_seq_len=context, device=device,
                          max_step_tokens=step_tokens, kernels=kernels))

    @classmethod
    def from_random(cls, config: Union[dict, object], seed: int, dtype: str = "bfloat16", context: Optional[int] = None,
                    batch: int = 8, device: str = "cuda:0", step_tokens: Optional[int] = None,
                    kernels: str = "fast") -> "Model":
        """Random weights for a configuration (a ``config.json`` dictionary or a configuration
        object of a registered architecture) and a seed."""
        import tempfile

        from ..config import config_from_json
        from ..weights.random_init import write_random_model

        cfg = config_from_json(config) if isinstance(config, dict) else config
        with tempfile.TemporaryDirectory(prefix="smolmoe_b200_") as tmp:
            write_random_model(cfg, tmp, seed)
            return cls.from_folder(tmp, dtype, context, batch, device, step_tokens, kernels)

    # ---- generating ----------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], tokens: int = 64, temperature: float = 0.0, top_k: int = 40,
                 top_p: float = 0.95, seed: int = 1, stop_ids: Optional[Iterable[int]] = None,
                 banned_ids: Iterable[int] = (), batch: Optional[int] = None, sink: Optional[TokenSink] = None,
                 return_completions: bool = False) -> Union[List[List[int]], List[Completion]]:
        """Generates up to ``tokens`` new token ids for each prompt (lists of token ids on the
        host). ``stop_ids`` defaults to the configuration's end-of-sequence ids; a stop token
        ends its sequence and is the last token returned for it."""
        engine = self.engine
        stops = tuple(stop_ids) if stop_ids is not None else tuple(engine.spec.stop_token_ids)
        for p in prompts:
            for t in p:
                if not 0 <= int(t) < engine.vocab_size:
                    raise ValueError(f"token {t} out of vocabulary ({engine.vocab_size})")
        sampler = Sampler(engine.runtime.ops, engine.vocab_size, SamplingOptions(temperature, top_k, top_p, seed),
                          engine.device, banned_ids)
        options = GenerationOptions(max_new_tokens=tokens, stop_token_ids=stops,
                                    batch=min(batch or engine.cache.max_slots, engine.cache.max_slots))
        self.last_stats = GenerationStats()
        done = generate(engine, sampler, prompts, options, sink, self.last_stats)
        engine.check_status()
        return done if return_completions else [c.tokens for c in done]

    def step(self, slots, tokens, want=None):
        """The engine's step function (see ``Engine.step``)."""
        return self.engine.step(slots, tokens, want)
