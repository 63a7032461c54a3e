"""What the C interface (``capi/engine.h``) calls: plain numbers and addresses in, the engine's own entry point
(``Model``) underneath. The C side holds no model state and computes nothing; this module reads the caller's arrays
through ctypes, calls ``Model.generate`` / ``Engine.step``, and writes results back to the caller's memory. The
reference's counterpart is the layer between its window and its engine (src/desktop.c over src/engine.c)."""
from __future__ import annotations

import ctypes
import json
from typing import List, Optional

from .generate import TokenSink


class _Request(ctypes.Structure):
    _fields_ = [("tokens", ctypes.POINTER(ctypes.c_int32)), ("n", ctypes.c_int32)]


class _Sink(ctypes.Structure):
    _fields_ = [("ctx", ctypes.c_void_p),
                ("token", ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32)),
                ("stop", ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p))]


class _CallerSink(TokenSink):
    """The caller's callbacks as the generation loop's sink (src/engine_sink.h:9-23)."""

    def __init__(self, address: int):
        self.sink = _Sink.from_address(address) if address else None

    def on_token(self, request: int, token: int, last: bool) -> None:
        if self.sink is not None and self.sink.token:
            self.sink.token(self.sink.ctx, request, token, int(last))

    def should_stop(self) -> bool:
        return bool(self.sink is not None and self.sink.stop and self.sink.stop(self.sink.ctx))


class Handle:
    def __init__(self, model, batch: int):
        self.model, self.batch = model, batch


def _open(make, options: dict) -> Handle:
    batch = int(options.get("batch") or 8)
    if batch < 0 or int(options.get("context") or 0) < 0 or int(options.get("step_tokens") or 0) < 0:
        raise ValueError("context, batch and step_tokens must not be negative")
    model = make(dtype=options.get("dtype") or "bfloat16", context=int(options.get("context") or 0) or None, batch=batch,
                 step_tokens=int(options.get("step_tokens") or 0) or None, kernels=options.get("kernels") or "fast")
    return Handle(model, batch)


def open_folder(folder: str, seed: int, options: dict) -> Handle:
    from .entry import Model
    return _open(lambda **kw: Model.from_folder(folder, **kw), options)


def open_random(config_json: str, seed: int, options: dict) -> Handle:
    from .entry import Model
    with open(config_json, "r", encoding="utf-8") as f:
        config = json.load(f)
    return _open(lambda **kw: Model.from_random(config, seed, **kw), options)


def close(handle: Handle) -> None:
    handle.model = None


def info(handle: Handle):
    engine, stats = handle.model.engine, handle.model.last_stats
    return (engine.vocab_size, engine.max_seq_len, handle.batch, len(engine.spec.order), engine.weight_bytes(),
            engine.cache.bytes_per_token() * engine.cache.max_tokens, stats.prompt_tokens if stats else 0,
            stats.generated_tokens if stats else 0, stats.prefill_seconds if stats else 0.0,
            stats.decode_seconds if stats else 0.0)


def generate(handle: Handle, requests: int, n: int, sink: int, tokens: int, temperature: float, top_k: int, top_p: float,
             seed: int, stop_ids: int, n_stop_ids: int) -> None:
    array = (_Request * n).from_address(requests)
    prompts: List[List[int]] = [list(array[i].tokens[:array[i].n]) for i in range(n)]
    stops: Optional[List[int]] = None
    if n_stop_ids >= 0:
        stops = list((ctypes.c_int32 * n_stop_ids).from_address(stop_ids)) if n_stop_ids else []
    handle.model.generate(prompts, tokens=tokens or 64, temperature=temperature, top_k=top_k, top_p=top_p or 0.95,
                          seed=seed or 1, stop_ids=stops, batch=handle.batch, sink=_CallerSink(sink))


def slot_alloc(handle: Handle) -> int:
    return handle.model.engine.open_sequence()


def slot_free(handle: Handle, slot: int) -> int:
    handle.model.engine.close_sequence(slot)
    return 0


def slot_length(handle: Handle, slot: int) -> int:
    engine = handle.model.engine
    if slot not in engine.cache.lengths:
        raise ValueError(f"slot {slot} is not open")
    return engine.length(slot)


def step(handle: Handle, slots: int, counts: int, n: int, tokens: int, want: int, logits: int) -> None:
    import torch
    engine = handle.model.engine
    slot_list = list((ctypes.c_int32 * n).from_address(slots))
    count_list = list((ctypes.c_int32 * n).from_address(counts))
    if any(c < 1 for c in count_list):
        raise ValueError("every sequence of a step brings at least one token")
    flat = (ctypes.c_int32 * sum(count_list)).from_address(tokens)
    token_lists, at = [], 0
    for c in count_list:
        token_lists.append(list(flat[at:at + c]))
        at += c
    wanted = list((ctypes.c_uint8 * n).from_address(want)) if want else [1] * n
    rows = engine.step(slot_list, token_lists, [[c - 1] if w else [] for c, w in zip(count_list, wanted)])
    engine.check_status()
    if rows is not None:
        if not logits:
            raise ValueError("logits are wanted and no place for them was given")
        host = rows.to("cpu", torch.float32).contiguous()
        ctypes.memmove(logits, host.data_ptr(), host.numel() * 4)
