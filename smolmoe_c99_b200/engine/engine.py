"""The engine: a model on one GPU with its cache, and the one step function everything
above it uses (generation, trace replay, benchmarks).

``step`` takes a batch of sequences that either all start (whole prompts of unequal
lengths, one step) or all go on by one token; it runs only the tokens it is given, as one
batch, from the cache that earlier steps left, and returns the logits at the wanted places.
The reference's counterpart is ``model_forward(tokens, n, pos0, mode)`` for its single
sequence (src/model.h:79-97, src/model.c:664-724).
"""
from __future__ import annotations

import os
import tempfile
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..cache import CacheFull, SequenceCache
from ..config import load_config
from ..kernels import get_ops
from ..parts import Runtime
from ..weights.loader import load_weights
from .batch import StepBatch, pack_step
from .model import DecoderModel, cache_needs, model_param_specs

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class StepError(ValueError):
    """The step's arguments cannot be run (bad token, unknown slot, no room)."""


class Engine:
    def __init__(self, model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16", *, max_tokens: int = 4096,
                 max_slots: Optional[int] = None, max_seq_len: Optional[int] = None, device: str = "cuda:0"):
        self.dtype = DTYPES[dtype] if isinstance(dtype, str) else dtype
        if self.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype must be bfloat16 or float32")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.config = load_config(model_dir)
        self.spec = self.config.model_spec()
        self.max_seq_len = min(self.spec.max_positions, max_seq_len or max_tokens, max_tokens)
        self.runtime = Runtime(dtype=self.dtype, device=self.device, ops=get_ops(), max_positions=self.max_seq_len)
        self.model = DecoderModel(self.spec, self.runtime)
        tensors = load_weights(model_dir, model_param_specs(self.spec), self.dtype, self.device)
        self.model.bind(tensors)
        self.cache = SequenceCache(cache_needs(self.spec), max_tokens=max_tokens,
                                   max_slots=max_slots if max_slots is not None else 256,
                                   max_seq_len=self.max_seq_len, dtype=self.dtype, device=self.device)
        self.vocab_size = self.spec.vocab_size
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)

    # ---- construction from random weights ------------------------------------------------
    @classmethod
    def from_random(cls, config, seed: int, dtype="bfloat16", **kwargs) -> "Engine":
        """Writes a model folder with random weights into a temporary folder and loads it."""
        from ..weights.random_init import write_random_model

        with tempfile.TemporaryDirectory(prefix="smolmoe_b200_") as tmp:
            write_random_model(config, tmp, seed)
            return cls(tmp, dtype, **kwargs)

    # ---- sequences -----------------------------------------------------------------------
    def open_sequence(self) -> int:
        """A free slot for a new sequence (length 0)."""
        return self.cache.alloc_slot()

    def close_sequence(self, slot: int) -> None:
        """Gives the slot and what it holds back."""
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step function ---------------------------------------------------------------
    def step(self, slots: Sequence[int], token_lists: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """Runs ``token_lists[i]`` as the next tokens of the sequence in ``slots[i]``.

        ``want[i]`` lists the places among these tokens whose logits are asked for (default:
        the last token of each sequence). Returns float32 ``[wanted, vocab]`` on the device in
        the order of the sequences and of ``want``, or None if nothing is wanted.
        """
        if len(slots) != len(token_lists) or (want is not None and len(want) != len(slots)):
            raise StepError("slots, token lists and wanted places must have one entry per sequence")
        if len(set(slots)) != len(slots):
            raise StepError("a slot appears twice in one step")
        starts = []
        for slot, toks in zip(slots, token_lists):
            if slot not in self.cache.lengths:
                raise StepError(f"slot {slot} is not open")
            for t in toks:
                if not 0 <= int(t) < self.vocab_size:  # src/model.c:673
                    raise StepError(f"token {t} out of vocabulary ({self.vocab_size})")
            starts.append(self.cache.length(slot))
        try:
            batch = pack_step(slots, starts, token_lists, self.device)
        except ValueError as e:
            raise StepError(str(e)) from None
        growth = {slot: n for slot, n in zip(slots, batch.seq_lens)}
        try:
            self.cache.reserve(growth)
        except CacheFull as e:
            raise StepError(f"token batch exceeds the cache: {e}") from None  # src/model.c:669-670
        self.cache.flush_tables()
        rows: List[int] = []
        first = 0
        for i, n in enumerate(batch.seq_lens):
            places = [n - 1] if want is None else list(want[i])
            for p in places:
                if not 0 <= p < n:
                    raise StepError(f"wanted place {p} is outside the {n} tokens of sequence {i}")
                rows.append(first + p)
            first += n
        want_rows = torch.tensor(rows, dtype=torch.int32).to(self.device) if rows else None
        logits = self.model.forward(batch, self.cache, want_rows, self._status)
        self.cache.advance(growth)
        return logits

    # ---- figures -------------------------------------------------------------------------
    def weight_bytes(self) -> int:
        return self.model.weight_bytes()
