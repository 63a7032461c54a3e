"""The engine: a model on one GPU with its cache, and the one step function everything
above it uses (generation, trace replay, benchmarks).

``step`` takes a batch of sequences, each with one or more next tokens that start at the
sequence's current length: whole prompts of unequal lengths, one token each, a prompt in
portions, a later message onto a live sequence, or any mix of these in one step. It runs only
the tokens it is given, as one batch, from the cache that earlier steps left, and returns the
logits at the wanted places. The reference's counterpart is ``model_forward(tokens, n, pos0,
mode)`` for its single sequence (src/model.h:79-97, src/model.c:664-690), which
``model_prefill`` calls portion by portion (src/model.c:714-724) and the conversation engine
calls for every later message on the cache the earlier ones left (src/engine.c:222-241).

Steps of one token per sequence are launch-bound, so their kernels are captured once per
batch size into a CUDA graph and replayed; the step's numbers (tokens, positions, slots)
live in fixed device buffers that are refilled before each replay.
"""
from __future__ import annotations

import tempfile
from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from ..cache import CacheFull, SequenceCache
from ..config import load_config
from ..kernels import get_ops
from ..parts import Runtime
from ..weights.loader import load_weights
from .batch import StepBatch, pack_step
from .model import DecoderModel, cache_needs, model_param_specs

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
SPAN_BUCKET = 256    # decode graphs are captured for key spans rounded up to this, doubling from there on
MAX_GRAPHS = 32
MAX_STEP_GRAPHS = 4  # captured steps of prompts (each keeps the activations of its tokens)


class StepError(ValueError):
    """The step's arguments cannot be run (bad token, unknown slot, no room)."""


def _capture(device, run):
    """``run()`` captured into a CUDA graph on a stream of its own: returns (graph, what run returned).

    ``torch.cuda.graph`` is not used: on entry it collects Python garbage and gives the allocator's cached blocks back
    to the driver, which took ~0.4 s with a few GB cached -- a stall in the middle of generation whenever a batch
    reaches a span for which no graph has been captured yet."""
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph.capture_begin()
        try:
            out = run()
        except BaseException:
            try:
                graph.capture_end()      # the stream must leave capture mode whatever happened
            except Exception:
                pass
            raise
        graph.capture_end()
    torch.cuda.current_stream().wait_stream(side)
    return graph, out


class _DecodeGraph:
    """One captured decode step for a batch size and key span."""

    def __init__(self, engine: "Engine", n_seqs: int, span: int):
        dev = engine.device
        self.meta = torch.zeros((4, n_seqs), dtype=torch.int32, device=dev)  # tokens, positions, slots, ends
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.rows = torch.arange(n_seqs, dtype=torch.int32, device=dev)
        self.batch = StepBatch(
            mode="decode", n_seqs=n_seqs, n_tokens=n_seqs, slots=[], seq_lens=[1] * n_seqs, max_seq_len=span,
            tokens=self.meta[0], positions=self.meta[1], token_slot=self.meta[2], token_end=self.meta[3],
            token_seq_start=self.rows, cu_seqlens=torch.arange(n_seqs + 1, dtype=torch.int32, device=dev),
            slot_ids=self.meta[2], seq_ends=self.meta[3], wants_every_row=True)
        # The step's numbers go up from pinned host memory, asynchronously. A few buffers take turns; an event says
        # when the copy that last read a buffer is done, so that it can be written again.
        self._staging = [torch.empty((4, n_seqs), dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._staged: List[Optional[torch.cuda.Event]] = [None] * len(self._staging)
        self._turn = 0

    def upload(self, first_row: int, rows: List[List[int]]) -> None:
        """``meta[first_row:first_row + len(rows)] = rows`` in stream order, through pinned memory."""
        i = self._turn
        self._turn = (i + 1) % len(self._staging)
        if self._staged[i] is not None:
            self._staged[i].synchronize()
        else:
            self._staged[i] = torch.cuda.Event()
        host = self._staging[i][first_row:first_row + len(rows)]
        host.copy_(torch.tensor(rows, dtype=torch.int32))
        self.meta[first_row:first_row + len(rows)].copy_(host, non_blocking=True)
        self._staged[i].record()

    def capture(self, engine: "Engine") -> None:
        """``meta`` must already hold a real step: the run before the capture loads kernels and
        sets function attributes, and it writes the same keys and values the replay will."""
        # Keys and values are written twice with the same numbers, which is harmless; a state of
        # fixed size would be advanced twice, so it is put back after the run.
        saved = [s.clone() for s in engine.cache.states]
        try:
            side = torch.cuda.Stream(device=engine.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                engine.model.forward(self.batch, engine.cache, self.rows, engine._status)
            torch.cuda.current_stream().wait_stream(side)
        finally:
            for state, before in zip(engine.cache.states, saved):
                state.copy_(before)
        # the graph is taken for captured only once the capture has gone through: a failed one leaves no
        # half-made graph behind that a later step could replay
        self.graph, self.logits = _capture(
            engine.device, lambda: engine.model.forward(self.batch, engine.cache, self.rows, engine._status))


class _StepGraph:
    """One captured step of prompts or prompt portions: the numbers of tokens of its sequences and the wanted rows
    are fixed, everything else (tokens, positions, slots, pages) is data that each replay brings.

    A small model's prompt step is ~200 launches of a few microseconds of device time each, and the host needs
    longer to issue them than the device to run them. A shape that comes again (every full portion of a long
    prompt fed in portions; a benchmark's prompt) is therefore captured the second time it is seen."""

    def __init__(self, engine: "Engine", rows: List[int]):
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.packed: Optional[torch.Tensor] = None
        self.batch: Optional[StepBatch] = None
        self.want_rows = torch.tensor(rows, dtype=torch.int32).to(engine.device) if rows else None

    def run(self, engine: "Engine", slots, starts, tokens, span: int) -> Optional[torch.Tensor]:
        batch = pack_step(slots, starts, tokens, engine.device, into=self.packed)
        # (kernels that size themselves by the longest sequence do so for the span the graph is kept for, not for
        # this step's own longest sequence)
        batch.max_seq_len = max(batch.max_seq_len, span)
        if self.graph is None:
            # (No run outside the capture first: the shape's first step ran kernel by kernel, which loaded the kernels
            # and set their attributes. Nothing runs during the capture, so the replay below is this step's one run.)
            self.packed, self.batch = batch.packed, batch
            self.graph, self.logits = _capture(
                engine.device, lambda: engine.model.forward(batch, engine.cache, self.want_rows, engine._status))
        self.graph.replay()
        return self.logits


class Engine:
    def __init__(self, model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16", *, max_tokens: int = 4096,
                 max_slots: Optional[int] = None, max_seq_len: Optional[int] = None, device: str = "cuda:0",
                 use_graphs: bool = True, max_step_tokens: Optional[int] = None, kernels: str = "fast"):
        self.dtype = DTYPES[dtype] if isinstance(dtype, str) else dtype
        if self.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype must be bfloat16 or float32")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.config = load_config(model_dir)
        self.spec = self.config.model_spec()
        self.max_seq_len = min(self.spec.max_positions, max_seq_len or max_tokens, max_tokens)
        self.runtime = Runtime(dtype=self.dtype, device=self.device, ops=get_ops(kernels), max_positions=self.max_seq_len)
        self.model = DecoderModel(self.spec, self.runtime)
        tensors = load_weights(model_dir, model_param_specs(self.spec), self.dtype, self.device)
        self.model.bind(tensors)
        self.cache = SequenceCache(cache_needs(self.spec), max_tokens=max_tokens,
                                   max_slots=max_slots if max_slots is not None else 256,
                                   max_seq_len=self.max_seq_len, dtype=self.dtype, device=self.device)
        self.vocab_size = self.spec.vocab_size
        self.use_graphs = use_graphs
        # a generation loop may launch the next one-token step before it has read the tokens just chosen (generate.py)
        self.runs_ahead = True
        # the most tokens one step may bring (all sequences together): it bounds a step's activations, as the
        # reference's --batch bounds its buffers (src/model.c:669); None: no bound but the cache's
        if max_step_tokens is not None and max_step_tokens < 1:
            raise ValueError("max_step_tokens must be at least 1")
        self.max_step_tokens = max_step_tokens
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._graphs: "OrderedDict[Tuple[int, int], _DecodeGraph]" = OrderedDict()
        # steps of prompts: how often a shape was seen, and the captured ones (a few: each keeps its activations)
        self._step_seen: "OrderedDict[tuple, int]" = OrderedDict()
        self._step_graphs: "OrderedDict[tuple, _StepGraph]" = OrderedDict()
        self.step_graph_max_tokens = 16384
        self._has_ring = any(group.ring > 0 for group in self.cache.groups)
        self.kernel_launches = 0   # graph replays and eager steps, for the record

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
    def step(self, slots: Sequence[int], tokens: Union[Sequence[Sequence[int]], torch.Tensor],
             want: Optional[Sequence[Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """Runs the next tokens of the sequences in ``slots``: sequence ``i`` brings ``len(tokens[i]) >= 1``
        tokens, which take the positions from its current length on. Sequences at their first token, sequences
        that go on by one token and sequences that go on by several may share a step.

        ``tokens`` is a list of token lists, one per sequence, or -- for a step of one token
        each -- an int32 device tensor ``[len(slots)]`` (what the sampler returned; it is not
        read back to the host). ``want[i]`` lists the places among sequence ``i``'s tokens
        whose logits are asked for (default: its last token). Returns float32
        ``[wanted, vocab]`` on the device in the order of the sequences and of ``want``, or
        None if nothing is wanted. The result may be overwritten by the next step.
        """
        n = len(slots)
        on_device = isinstance(tokens, torch.Tensor)
        if on_device:
            if tokens.dtype != torch.int32 or tokens.dim() != 1 or tokens.numel() != n or not tokens.is_cuda:
                raise StepError("device tokens must be an int32 CUDA tensor with one token per sequence")
            lens = [1] * n
        else:
            if len(tokens) != n:
                raise StepError("slots and token lists must have one entry per sequence")
            lens = [len(t) for t in tokens]
            for toks in tokens:
                if len(toks) and not (0 <= min(toks) and max(toks) < self.vocab_size):  # src/model.c:673
                    bad = next(t for t in toks if not 0 <= int(t) < self.vocab_size)
                    raise StepError(f"token {bad} out of vocabulary ({self.vocab_size})")
        if n == 0 or any(k == 0 for k in lens):
            raise StepError("a step needs at least one sequence, and every sequence at least one token")
        if want is not None and len(want) != n:
            raise StepError("wanted places must have one entry per sequence")
        if len(set(slots)) != n:
            raise StepError("a slot appears twice in one step")
        for slot in slots:
            if slot not in self.cache.lengths:
                raise StepError(f"slot {slot} is not open")
        starts = [self.cache.length(slot) for slot in slots]
        rows: List[int] = []
        first = 0
        for i, k in enumerate(lens):
            for p in ([k - 1] if want is None else want[i]):
                if not 0 <= p < k:
                    raise StepError(f"wanted place {p} is outside the {k} tokens of sequence {i}")
                rows.append(first + p)
            first += k
        if self.max_step_tokens is not None and sum(lens) > self.max_step_tokens:   # src/model.c:669
            raise StepError(f"the step brings {sum(lens)} tokens, more than max_step_tokens = {self.max_step_tokens}: "
                            f"feed the prompts in portions")
        decode = all(k == 1 for k in lens) and all(s > 0 for s in starts)
        growth = {slot: k for slot, k in zip(slots, lens)}
        try:
            self.cache.reserve(growth)
        except CacheFull as e:
            raise StepError(f"token batch exceeds the cache: {e}") from None  # src/model.c:669-670
        self.cache.flush_tables()
        if decode and self.use_graphs:
            logits = self._decode_graph(slots, starts, tokens, on_device)
            if rows != list(range(n)):
                logits = logits[torch.tensor(rows, dtype=torch.long, device=self.device)] if rows else None
        else:
            if on_device:
                tokens = [[int(t)] for t in tokens.tolist()]
            logits = self._prompt_step(slots, starts, tokens, lens, rows)
        self.kernel_launches += 1
        self.cache.advance(growth)
        return logits

    def _prompt_step(self, slots, starts, tokens, lens, rows) -> Optional[torch.Tensor]:
        """A step that is not one token each: eagerly, or -- a shape seen before -- as a captured graph."""
        first = all(s == 0 for s in starts)
        # (a windowed group's late store and the check of its ring are decided on the host from the starts: those
        # steps stay eager unless every sequence is at its first token)
        if self.use_graphs and sum(lens) <= self.step_graph_max_tokens and (first or not self._has_ring):
            # Sequences that go on from the cache: the longest of them after the step, rounded up the way the decode
            # graphs' spans are, is part of the shape (the attention over the cache is launched for it).
            span = 0
            if not first:
                longest = max(s + n for s, n in zip(starts, lens))
                span = SPAN_BUCKET
                while span < longest:
                    span *= 2
                span = min(span, -(-self.max_seq_len // 128) * 128)
            key = (first, tuple(lens), tuple(rows), span)
            g = self._step_graphs.get(key)
            if g is None:
                seen = self._step_seen.pop(key, 0) + 1
                self._step_seen[key] = seen
                while len(self._step_seen) > 64:
                    self._step_seen.popitem(last=False)
                if seen >= 2:
                    while len(self._step_graphs) >= MAX_STEP_GRAPHS:
                        self._step_graphs.popitem(last=False)
                    g = self._step_graphs[key] = _StepGraph(self, rows)
            else:
                self._step_graphs.move_to_end(key)
            if g is not None:
                try:
                    return g.run(self, slots, starts, tokens, span)
                except BaseException:
                    self._step_graphs.pop(key, None)
                    raise
        batch = pack_step(slots, starts, tokens, self.device)
        want_rows = torch.tensor(rows, dtype=torch.int32).to(self.device) if rows else None
        return self.model.forward(batch, self.cache, want_rows, self._status)

    def _decode_graph(self, slots, starts, tokens, on_device) -> torch.Tensor:
        n = len(slots)
        longest = max(starts) + 1
        span = SPAN_BUCKET
        while span < longest:
            span *= 2   # a capture costs tens of steps: few spans, each good for as many steps as came before it
        span = min(span, -(-self.max_seq_len // 128) * 128)
        key = (n, span)
        g = self._graphs.get(key)
        if g is None:
            if len(self._graphs) >= MAX_GRAPHS:
                self._graphs.popitem(last=False)
            g = self._graphs[key] = _DecodeGraph(self, n, span)
        else:
            self._graphs.move_to_end(key)
        g.upload(0, [[0] * n if on_device else [int(t[0]) for t in tokens], list(starts), list(slots),
                     [s + 1 for s in starts]])
        if on_device:
            g.meta[0].copy_(tokens)
        if g.graph is None:
            try:
                g.capture(self)
            except BaseException:
                self._graphs.pop(key, None)
                raise
        g.graph.replay()
        return g.logits

    # ---- a one-token step in two halves ----------------------------------------------------
    def prepare_decode(self, slots: Sequence[int]):
        """The host's share of the next one-token step of ``slots`` that does not depend on the tokens:
        room in the cache, and the step's positions and slots copied into the captured graph's buffers
        (in stream order, so behind the step that may still be running). A generation loop calls this
        before it waits for the tokens it has just chosen, and ``launch_prepared`` after. Returns None where
        the plain ``step`` has to do it (no graphs, a graph still to be captured, a sequence at its start)."""
        n = len(slots)
        if not self.use_graphs or n == 0 or len(set(slots)) != n or any(s not in self.cache.lengths for s in slots):
            return None
        starts = [self.cache.length(slot) for slot in slots]
        if min(starts) == 0:
            return None
        longest = max(starts) + 1
        span = SPAN_BUCKET
        while span < longest:
            span *= 2
        span = min(span, -(-self.max_seq_len // 128) * 128)
        g = self._graphs.get((n, span))
        if g is None or g.graph is None:
            return None
        try:
            self.cache.reserve({slot: 1 for slot in slots})
        except CacheFull:
            return None
        self.cache.flush_tables()
        self._graphs.move_to_end((n, span))
        g.upload(1, [list(starts), list(slots), [s + 1 for s in starts]])
        return g, tuple(slots), tuple(starts)

    def launch_prepared(self, prepared, tokens: torch.Tensor) -> torch.Tensor:
        """Runs the step that ``prepare_decode`` prepared, with one int32 device token per sequence; returns
        the logits of every sequence like ``step``."""
        g, slots, starts = prepared
        if tokens.dtype != torch.int32 or tokens.dim() != 1 or tokens.numel() != len(slots) or not tokens.is_cuda:
            raise StepError("device tokens must be an int32 CUDA tensor with one token per sequence")
        if tuple(self.cache.lengths.get(slot, -1) for slot in slots) != starts:
            raise StepError("the sequences changed between prepare_decode and launch_prepared")
        g.meta[0].copy_(tokens)
        g.graph.replay()
        self.kernel_launches += 1
        self.cache.advance({slot: 1 for slot in slots})
        return g.logits

    def synchronize(self) -> None:
        torch.cuda.synchronize(self.device)

    # ---- time per phase --------------------------------------------------------------------
    def start_profile(self) -> None:
        """From now on the device time of every step is charged to the reference's phases (src/model.c:312-328).
        Steps then run kernel by kernel, without graphs (an event cannot be timed inside one); what they compute
        is unchanged."""
        from ..kernels.ops import PhaseTimes
        self._graphs_before_profile = self.use_graphs
        self.use_graphs = False
        self.runtime.ops.phase_times = PhaseTimes()

    def stop_profile(self) -> Dict[str, float]:
        """Seconds per phase since ``start_profile`` (synchronises)."""
        times = self.runtime.ops.phase_times
        self.runtime.ops.phase_times = None
        self.use_graphs = getattr(self, "_graphs_before_profile", self.use_graphs)
        return times.seconds() if times is not None else {}

    def check_status(self) -> None:
        """Raises if a kernel reported a fault since the last check (synchronises)."""
        self.runtime.ops.check_error_flag()
        if int(self._status.item()):
            self._status.zero_()
            raise StepError("a token outside the vocabulary reached the device")

    # ---- figures -------------------------------------------------------------------------
    def weight_bytes(self) -> int:
        return self.model.weight_bytes()
