"""One step's work as the kernels see it: the tokens of all sequences packed one after
another, with each token's position, slot and sequence.

Every sequence brings ``n_i >= 1`` tokens that start at its current length (the reference's
``model_forward(tokens, n, pos0)``, src/model.c:664-690, for many sequences at once). Two
shapes of a step have kernels of their own and are told apart by ``mode``: ``prefill`` (every
sequence starts at its first token: whole prompts of unequal lengths) and ``decode`` (every
sequence goes on by one token). Everything else is ``extend``: prompts in portions, a later
message onto a live sequence, new sequences joining ones that decode."""
from __future__ import annotations

from dataclasses import dataclass
from array import array
from typing import List, Optional, Sequence

import torch


QUERY_TILE = 64  # queries per CTA of the prefill attention kernel


@dataclass
class StepBatch:
    mode: str                       # "prefill", "decode" or "extend"
    n_seqs: int
    n_tokens: int
    slots: List[int]                # per sequence
    seq_lens: List[int]             # tokens of each sequence in this step
    max_seq_len: int                # longest sequence after this step
    tokens: torch.Tensor            # int32 [T]
    positions: torch.Tensor         # int32 [T] absolute positions
    token_slot: torch.Tensor        # int32 [T]
    token_end: torch.Tensor         # int32 [T] the token's sequence length after this step
    token_seq_start: torch.Tensor   # int32 [T] packed index of the sequence's first token
    cu_seqlens: torch.Tensor        # int32 [B + 1]
    slot_ids: torch.Tensor          # int32 [B]
    seq_ends: torch.Tensor          # int32 [B] lengths after this step
    prefill_tiles: Optional[torch.Tensor] = None  # int32 [tiles, 3]: sequence's first packed index, length, first query
    extend_tiles: Optional[torch.Tensor] = None   # int32 [tiles, 5]: first packed index, tokens in this step, first query
                                                  # among them, position of the step's first token, slot
    seq_starts: Optional[List[int]] = None        # per sequence: its length before this step
    wants_every_row: bool = False   # logits are asked for every token of the step, in order
    packed: Optional[torch.Tensor] = None         # the one device buffer that the tensors above are views of


def pack_step(slots: Sequence[int], starts: Sequence[int], token_lists: Sequence[Sequence[int]],
              device: torch.device, into: Optional[torch.Tensor] = None) -> StepBatch:
    """``starts[i]`` is the length of sequence ``i`` before this step. ``into``: a device buffer that a step of the
    same shape (the same numbers of tokens) was packed into before; the step's numbers are copied there, so that
    kernels captured in a graph find them where they found the earlier step's."""
    if not slots:
        raise ValueError("a step needs at least one sequence")
    lens = [len(t) for t in token_lists]
    if any(n == 0 for n in lens):
        raise ValueError("every sequence of a step brings at least one token")
    if any(s < 0 for s in starts) or len(starts) != len(slots) or len(lens) != len(slots):
        raise ValueError("every sequence of a step needs a slot, a start that is not negative and its tokens")
    if all(s == 0 for s in starts):
        mode = "prefill"
    elif all(n == 1 for n in lens) and all(s > 0 for s in starts):
        mode = "decode"
    else:
        mode = "extend"
    # the step's numbers, one row per quantity, built with tensor operations (a prompt of thousands of tokens
    # would spend a millisecond in Python loops otherwise)
    n_seqs = len(slots)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    n_tokens = cu[-1]
    # everything the device needs of this step goes up in ONE copy: five rows of n_tokens numbers, then the
    # prefill tiles, the slots, the sequences' ends and the sequences' first packed indices
    tile_rows: List[List[int]] = []
    if mode == "prefill":
        tile_rows = [[cu[i], n, q0] for i, n in enumerate(lens) for q0 in range(0, n, QUERY_TILE)]
    elif mode == "extend":
        tile_rows = [[cu[i], n, q0, starts[i], slots[i]] for i, n in enumerate(lens) for q0 in range(0, n, QUERY_TILE)]
    tile_width = 3 if mode == "prefill" else 5
    extra = tile_width * len(tile_rows) + 2 * n_seqs + (n_seqs + 1)
    # (pinned memory on a GPU box: the copy below is then asynchronous and the allocator keeps the buffer until it is done)
    flat_host = torch.empty(5 * n_tokens + extra, dtype=torch.int32, pin_memory=device.type == "cuda")
    host = flat_host[:5 * n_tokens].view(5, n_tokens)
    flat = token_lists[0] if n_seqs == 1 else [t for toks in token_lists for t in toks]
    host[0] = torch.frombuffer(array("i", flat), dtype=torch.int32) if n_tokens else host[0]
    if n_seqs <= 4:
        for i, (slot, start, n) in enumerate(zip(slots, starts, lens)):
            a, b = cu[i], cu[i + 1]
            torch.arange(start, start + n, dtype=torch.int32, out=host[1, a:b])
            host[2, a:b] = slot
            host[3, a:b] = start + n
            host[4, a:b] = a
    else:
        lens_t = torch.tensor(lens, dtype=torch.int32)
        starts_t = torch.tensor(list(starts), dtype=torch.int32)
        firsts = torch.tensor(cu[:-1], dtype=torch.int32)
        seq_of = torch.repeat_interleave(torch.arange(n_seqs), lens_t.long())
        host[1] = torch.arange(n_tokens, dtype=torch.int32) - firsts[seq_of] + starts_t[seq_of]
        host[2] = torch.tensor(list(slots), dtype=torch.int32)[seq_of]
        host[3] = (starts_t + lens_t)[seq_of]
        host[4] = firsts[seq_of]
    tail = [x for row in tile_rows for x in row] + list(slots) + [s + n for s, n in zip(starts, lens)] + cu
    flat_host[5 * n_tokens:] = torch.tensor(tail, dtype=torch.int32)
    if into is None:
        flat_dev = flat_host.to(device, non_blocking=True)
    else:
        if into.numel() != flat_host.numel() or into.dtype != torch.int32:
            raise ValueError("the buffer was packed for a step of another shape")
        into.copy_(flat_host, non_blocking=True)
        flat_dev = into
    dev = flat_dev[:5 * n_tokens].view(5, n_tokens)
    at = 5 * n_tokens
    tiles = None
    if tile_rows:
        tiles = flat_dev[at:at + tile_width * len(tile_rows)].view(len(tile_rows), tile_width)
        at += tile_width * len(tile_rows)
    per_seq = flat_dev[at:at + 2 * n_seqs].view(2, n_seqs)
    cu_dev = flat_dev[at + 2 * n_seqs:at + 3 * n_seqs + 1]
    return StepBatch(
        mode=mode, n_seqs=len(slots), n_tokens=n_tokens, slots=list(slots), seq_lens=lens,
        max_seq_len=max(s + n for s, n in zip(starts, lens)),
        tokens=dev[0], positions=dev[1], token_slot=dev[2], token_end=dev[3], token_seq_start=dev[4],
        cu_seqlens=cu_dev, slot_ids=per_seq[0], seq_ends=per_seq[1],
        prefill_tiles=tiles if mode == "prefill" else None, extend_tiles=tiles if mode == "extend" else None,
        seq_starts=list(starts), packed=flat_dev)
