"""The generation loop above the step function: batches of unequal prompts, stop tokens,
sequences that end earlier, and as many batches one after another as there are requests.

The reference's loop serves one prompt (src/main.c:571-600; chat: src/engine.c:149-219);
what carries over: the prompts go through in one step (or, where the engine bounds a
step's tokens, in portions as src/main.c:553-568 cuts them), then one token a step; a stop
token ends the sequence, is reported and is not fed back; the last token that the limit
allows is not fed back either (src/main.c:590); prompt plus new tokens must fit the context
(src/main.c:795-796); a sink receives every token and may ask to stop (src/engine_sink.h).
The loop only decides; the engine and the sampler it is given do the work, so it runs
unchanged over a stand-in engine in tests.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class GenerationOptions:
    max_new_tokens: int = 64            # --tokens (src/main.c:29)
    stop_token_ids: Tuple[int, ...] = ()
    batch: int = 8                      # sequences that start together


@dataclass
class Completion:
    prompt_tokens: int
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""             # "stop", "length" or "cancelled"


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    decode_forwards: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    ttft_seconds: float = 0.0           # from the start of the call to the first batch's first logits
    batches: int = 0

    def as_dict(self) -> Dict[str, float]:
        """The reference's keys and definitions (src/main.c:347-382)."""
        return {
            "prompt_tokens": self.prompt_tokens, "generated_tokens": self.generated_tokens,
            "processed_tokens": self.prompt_tokens + self.decode_forwards, "ttft_seconds": self.ttft_seconds,
            "prefill_seconds": self.prefill_seconds, "decode_seconds": self.decode_seconds,
            "prefill_tokens_per_second": self.prompt_tokens / self.prefill_seconds if self.prefill_seconds > 0 else 0.0,
            "decode_tokens_per_second": self.decode_forwards / self.decode_seconds if self.decode_seconds > 0 else 0.0,
            "batches": self.batches,
        }


def prompt_portions(lengths: Sequence[int], limit: Optional[int]) -> List[List[Tuple[int, int, int]]]:
    """How the prompts of a batch go through when one step may bring at most ``limit`` tokens: a list of steps,
    each a list of ``(index, begin, end)`` -- prompt ``index`` brings its tokens ``begin:end``. Prompts are taken in
    order and every step is filled as far as the limit allows; without a limit, or when all prompts fit in it,
    there is one step with every prompt whole. The reference cuts its single prompt the same way into portions
    of ``--batch`` tokens (src/main.c:553-568)."""
    if limit is None or sum(lengths) <= limit:
        return [[(i, 0, n) for i, n in enumerate(lengths)]]
    if limit < 1:
        raise ValueError("a step must be allowed at least one token")
    steps: List[List[Tuple[int, int, int]]] = [[]]
    room = limit
    for i, n in enumerate(lengths):
        at = 0
        while at < n:
            if room == 0:
                steps.append([])
                room = limit
            take = min(n - at, room)
            steps[-1].append((i, at, at + take))
            at += take
            room -= take
    return steps


def _start_read(chosen, buffer: dict):
    """Asks for the chosen tokens on the host without waiting: a copy into pinned memory and an event behind it.
    Tensors that are on the host already (a stand-in engine) are handed through."""
    if not getattr(chosen, "is_cuda", False):
        return chosen, None
    import torch

    n = chosen.numel()
    if buffer.get("host") is None or buffer["host"].numel() < n:
        buffer["host"] = torch.empty(max(n, 64), dtype=chosen.dtype, pin_memory=True)
        buffer["event"] = torch.cuda.Event()
    host = buffer["host"][:n]
    host.copy_(chosen, non_blocking=True)
    buffer["event"].record()
    return host, buffer["event"]


def _finish_read(reading) -> List[int]:
    host, event = reading
    if event is not None:
        event.synchronize()
    return [int(t) for t in host.tolist()]


def _run_prompts(engine, slots: List[int], prompts: List[Sequence[int]]):
    """Feeds the prompts in as few steps as the engine's ``max_step_tokens`` allows and returns the logits after
    each prompt's last token, one row per prompt in order."""
    plan = prompt_portions([len(p) for p in prompts], getattr(engine, "max_step_tokens", None))
    if len(plan) == 1:
        return engine.step(slots, [list(p) for p in prompts])
    rows: List = [None] * len(prompts)
    for portion in plan:
        want = [[e - b - 1] if e == len(prompts[i]) else [] for i, b, e in portion]
        logits = engine.step([slots[i] for i, _, _ in portion], [list(prompts[i][b:e]) for i, b, e in portion], want)
        at = 0
        for (i, _, _), w in zip(portion, want):
            if w:
                rows[i] = logits[at:at + 1].clone()   # the next step may write over the engine's result
                at += 1
    import torch

    return torch.cat(rows, dim=0)


class TokenSink:
    """Receives tokens as they are chosen. ``should_stop`` is asked once per step."""

    def on_token(self, request: int, token: int, last: bool) -> None:
        pass

    def should_stop(self) -> bool:
        return False


def generate(engine, sampler, prompts: Sequence[Sequence[int]], options: GenerationOptions,
             sink: Optional[TokenSink] = None, stats: Optional[GenerationStats] = None,
             clock: Callable[[], float] = time.perf_counter) -> List[Completion]:
    """``engine`` provides open_sequence/close_sequence/step/max_seq_len/synchronize;
    ``sampler`` provides new_states/choose. Returns one completion per prompt, in order."""
    if options.batch <= 0 or options.max_new_tokens < 0:
        raise ValueError("batch must be positive and max_new_tokens must not be negative")
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"prompt {i} is empty")
        if len(p) + options.max_new_tokens > engine.max_seq_len:
            raise ValueError(f"prompt {i}: {len(p)} prompt tokens and {options.max_new_tokens} new tokens "
                             f"exceed the context of {engine.max_seq_len}")
    sink = sink or TokenSink()
    stats = stats if stats is not None else GenerationStats()
    stop = set(options.stop_token_ids)
    results = [Completion(prompt_tokens=len(p)) for p in prompts]
    cancelled = False
    read_buffer: dict = {}     # pinned memory for the chosen tokens on their way to the host
    for first in range(0, len(prompts), options.batch):
        ids = list(range(first, min(first + options.batch, len(prompts))))
        if cancelled or options.max_new_tokens == 0:
            for r in ids:
                results[r].finish_reason = "cancelled" if cancelled else "length"
            continue
        slots = {r: engine.open_sequence() for r in ids}
        live = list(ids)
        try:
            stats.batches += 1
            t0 = clock()
            logits = _run_prompts(engine, [slots[r] for r in live], [prompts[r] for r in live])
            states = sampler.new_states(live)
            engine.synchronize()
            t1 = clock()
            stats.prefill_seconds += t1 - t0
            if stats.batches == 1:
                stats.ttft_seconds = t1 - t0
            stats.prompt_tokens += sum(len(prompts[r]) for r in live)
            for produced in range(1, options.max_new_tokens + 1):
                chosen = sampler.choose(logits, states)
                # while the choice is still being computed: the host's share of the next step that does not
                # depend on it (an engine may offer this; it is redone the plain way if the batch changes)
                prepared = None
                if produced < options.max_new_tokens and hasattr(engine, "prepare_decode"):
                    prepared = engine.prepare_decode([slots[r] for r in live])
                # An engine that takes the chosen tokens on the device can be given the next step before the host has
                # read them (``runs_ahead``): the GPU then never waits for the host. A sequence that turns out to have
                # ended with this token has taken one step too many, into a slot that is closed below; no result
                # depends on it (a row's logits do not depend on what else is in the batch) and its row is dropped.
                ahead = None
                if prepared is not None and getattr(engine, "runs_ahead", False):
                    # the read of the chosen tokens is asked for BEFORE the next step is launched (a read asked for
                    # after it would wait behind it in the stream), and waited for after
                    reading = _start_read(chosen, read_buffer)
                    ahead = engine.launch_prepared(prepared, chosen)
                    tokens = _finish_read(reading)
                else:
                    tokens = [int(t) for t in chosen.tolist()]   # the one device-to-host read of the step
                keep = []
                for i, r in enumerate(live):
                    tok = tokens[i]
                    if tok < 0:
                        raise RuntimeError("every token is banned")  # src/sampler.c:61
                    results[r].tokens.append(tok)
                    stats.generated_tokens += 1
                    done = "stop" if tok in stop else ("length" if produced == options.max_new_tokens else "")
                    sink.on_token(r, tok, bool(done))
                    if done:
                        results[r].finish_reason = done
                        engine.close_sequence(slots.pop(r))
                    else:
                        keep.append(i)
                if sink.should_stop():
                    cancelled = True
                    for i in keep:
                        results[live[i]].finish_reason = "cancelled"
                    break
                if not keep:
                    break
                shrunk = len(keep) != len(live)
                if shrunk:   # shorter requests have ended: the batch shrinks
                    chosen, states = sampler.select(chosen, keep), sampler.select(states, keep)
                    live = [live[i] for i in keep]
                if ahead is not None:
                    logits = sampler.select(ahead, keep) if shrunk else ahead
                elif prepared is not None and not shrunk:
                    logits = engine.launch_prepared(prepared, chosen)
                else:
                    logits = engine.step([slots[r] for r in live], chosen)
                stats.decode_forwards += len(live)
            engine.synchronize()
            stats.decode_seconds += clock() - t1
        finally:
            for slot in slots.values():
                engine.close_sequence(slot)
    return results
