"""The cache: a slot for each sequence of a batch, keys and values for each layer that keeps
them, each sequence with its own length, and beside it per-sequence state of fixed size.

Storage is handed out in pages of ``PAGE_SIZE`` positions. Layers with the same need (kv
heads, head size, all keys or a window of them) form a group; every group has its own
pools, its own page table and its own page ledger. A windowed group keeps a ring of the
last ``ring`` positions (the window rounded up to whole pages): position ``p`` lives at ring
index ``p % ring``. The reference keeps one flat ``[layers][context][kv_dim]`` buffer for its
single sequence, and full-context storage even for windowed layers
(src/model.c:177-181,465-472).

Pool layout (one per layer of a group): ``[pages, kv_heads, PAGE_SIZE, head_dim]``.
Page table (one per group): ``int32 [slots, pages_per_sequence]``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from ..kernels.ops import PAGE_SIZE   # one number for host and kernels; the library's own is checked when it is loaded
from ..parts.base import KVNeed, StateNeed
from .allocators import CacheFull, CacheStateError, PageAllocator, SlotAllocator


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_SIZE - 1) // PAGE_SIZE


@dataclass
class LayerCache:
    """What one run of a layer sees of the cache."""

    kind: str  # "kv", "state" or "none"
    k_pool: Optional[torch.Tensor] = None
    v_pool: Optional[torch.Tensor] = None
    page_table: Optional[torch.Tensor] = None
    ring: int = 0
    window: Optional[int] = None
    state: Optional[torch.Tensor] = None  # [slots, *shape]


class KVGroup:
    def __init__(self, need: KVNeed, n_layers: int, n_pages: int, n_slots: int, max_seq_len: int,
                 dtype: torch.dtype, device: torch.device):
        self.need = need
        self.ring = pages_for(need.window) * PAGE_SIZE if need.window else 0
        self.pages_per_seq = pages_for(self.ring if self.ring else max_seq_len)
        self.ledger = PageAllocator(n_pages)
        shape = (n_layers, n_pages, need.kv_heads, PAGE_SIZE, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.table = torch.zeros((n_slots, self.pages_per_seq), dtype=torch.int32, device=device)
        self.slot_pages: Dict[int, List[int]] = {}
        self.n_layers = n_layers

    def pages_needed(self, length: int) -> int:
        n = pages_for(length)
        return min(n, self.pages_per_seq) if self.ring else n

    def bytes_per_token(self) -> int:
        return 2 * self.n_layers * self.need.kv_heads * self.need.head_dim * self.k.element_size()


class SequenceCache:
    """Built from what each run of a layer needs, in run order: a ``KVNeed``, a
    ``StateNeed``, ``None``, or an int naming the earlier run whose cache it reads."""

    def __init__(self, needs: Sequence[Union[KVNeed, StateNeed, None, int]], *, max_tokens: int, max_slots: int,
                 max_seq_len: int, dtype: torch.dtype, device: Union[str, torch.device]):
        if max_tokens <= 0 or max_seq_len <= 0:
            raise ValueError("max_tokens and max_seq_len must be positive")
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_tokens = max_tokens
        self.max_seq_len = max_seq_len
        self.n_pages = pages_for(max_tokens)
        self.max_slots = max(1, min(max_slots, self.n_pages))
        self.slots = SlotAllocator(self.max_slots)
        self.lengths: Dict[int, int] = {}
        self.groups: List[KVGroup] = []
        self._run_view: List[Tuple[str, int, int]] = []  # per run: (kind, group/state index, layer index in group)
        self.states: List[torch.Tensor] = []
        group_of: Dict[KVNeed, int] = {}
        members: Dict[int, int] = {}
        plan: List[Tuple[str, object, int]] = []
        for run, need in enumerate(needs):
            if isinstance(need, KVNeed):
                if need.head_dim % 8:
                    raise ValueError(f"run {run}: head_dim {need.head_dim} must be a multiple of 8")
                g = group_of.setdefault(need, len(group_of))
                plan.append(("kv", g, members.get(g, 0)))
                members[g] = members.get(g, 0) + 1
            elif isinstance(need, StateNeed):
                plan.append(("state", need, 0))
            elif need is None:
                plan.append(("none", None, 0))
            elif isinstance(need, int):
                if not 0 <= need < run or isinstance(needs[need], int) or needs[need] is None:
                    raise ValueError(f"run {run} reads the cache of run {need}, which owns none before it")
                plan.append(("shared", need, 0))
            else:
                raise TypeError(f"run {run}: unknown cache need {need!r}")
        for need, g in sorted(group_of.items(), key=lambda kv: kv[1]):
            self.groups.append(KVGroup(need, members[g], self.n_pages, self.max_slots, max_seq_len, dtype, self.device))
        for kind, what, index in plan:
            if kind == "kv":
                self._run_view.append(("kv", what, index))
            elif kind == "state":
                self.states.append(torch.zeros((self.max_slots, *what.shape), dtype=what.dtype, device=self.device))
                self._run_view.append(("state", len(self.states) - 1, 0))
            elif kind == "none":
                self._run_view.append(("none", 0, 0))
            else:
                self._run_view.append(self._run_view[what])
        self._dirty: Dict[int, set] = {g: set() for g in range(len(self.groups))}

    # ---- slots -------------------------------------------------------------------------
    def alloc_slot(self) -> int:
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        for g in self.groups:
            g.slot_pages[slot] = []
        for s in self.states:
            s[slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        if slot not in self.lengths:
            raise CacheStateError(f"slot {slot} is not held (freed twice, or never given out)")
        for g in self.groups:
            g.ledger.free(g.slot_pages.pop(slot))
        del self.lengths[slot]
        self.slots.free(slot)

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    # ---- growth ------------------------------------------------------------------------
    def reserve(self, growth: Dict[int, int]) -> None:
        """Makes room for ``growth[slot]`` more positions in each named slot, in every
        group, or changes nothing and raises ``CacheFull``."""
        want: List[Tuple[int, KVGroup, int, int]] = []
        for slot, n in growth.items():
            if slot not in self.lengths:
                raise CacheStateError(f"slot {slot} is not held")
            new_len = self.lengths[slot] + n
            if n < 0 or new_len > self.max_seq_len:
                raise CacheFull(f"slot {slot}: {new_len} positions exceed the longest sequence of {self.max_seq_len}")
        for gi, g in enumerate(self.groups):
            need_pages = 0
            for slot, n in growth.items():
                extra = g.pages_needed(self.lengths[slot] + n) - len(g.slot_pages[slot])
                if extra > 0:
                    want.append((gi, g, slot, extra))
                    need_pages += extra
            if need_pages > g.ledger.free_count:
                raise CacheFull(f"{need_pages} pages of {PAGE_SIZE} positions asked for, {g.ledger.free_count} of "
                                f"{g.ledger.count} free (the cache holds {self.max_tokens} tokens)")
        for gi, g, slot, extra in want:
            pages = g.ledger.alloc(extra)
            g.slot_pages[slot].extend(pages)
            self._dirty[gi].add(slot)

    def advance(self, growth: Dict[int, int]) -> None:
        for slot, n in growth.items():
            self.lengths[slot] += n

    def truncate(self, slot: int, length: int) -> None:
        """Positions at and beyond ``length`` are dead; their pages stay with the slot."""
        if not 0 <= length <= self.lengths[slot]:
            raise CacheStateError(f"slot {slot}: cannot truncate {self.lengths[slot]} positions to {length}")
        if any(g.ring for g in self.groups) and length < self.lengths[slot]:
            raise CacheStateError("a windowed group has dropped older positions: truncation is not possible")
        if self.states and length < self.lengths[slot]:
            raise CacheStateError("a state of fixed size cannot be rolled back")
        self.lengths[slot] = length

    def flush_tables(self) -> None:
        """Copies the page-table rows that changed to the device (on the current stream)."""
        for gi, slots in self._dirty.items():
            g = self.groups[gi]
            for slot in sorted(slots):
                row = g.slot_pages[slot]
                if row:
                    g.table[slot, : len(row)].copy_(torch.tensor(row, dtype=torch.int32))
            slots.clear()

    # ---- views -------------------------------------------------------------------------
    def run_view(self, run: int) -> LayerCache:
        kind, index, layer = self._run_view[run]
        if kind == "kv":
            g = self.groups[index]
            return LayerCache("kv", g.k[layer], g.v[layer], g.table, g.ring, g.need.window)
        if kind == "state":
            return LayerCache("state", state=self.states[index])
        return LayerCache("none")

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.groups)

    def live_tokens_rounded(self) -> int:
        return sum(pages_for(n) * PAGE_SIZE for n in self.lengths.values())
