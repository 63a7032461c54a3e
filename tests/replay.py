"""Ways of cutting the same requests into steps, driven through the engine's step function.
Each returns ``{request id: float32 logits [length, vocab] on the CPU}`` for every position."""
from typing import Dict, List, Sequence

import torch


def whole(engine, requests: Dict[str, Sequence[int]]) -> Dict[str, torch.Tensor]:
    """Each request alone, its whole sequence in one step."""
    out = {}
    for rid, toks in requests.items():
        slot = engine.open_sequence()
        out[rid] = engine.step([slot], [toks], [list(range(len(toks)))]).cpu()
        engine.close_sequence(slot)
    return out


def tail_decoded(engine, requests: Dict[str, Sequence[int]], tail: int = 32) -> Dict[str, torch.Tensor]:
    """Each request alone: its beginning in one step, the last ``tail`` tokens one by one."""
    out = {}
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        slot = engine.open_sequence()
        rows = [engine.step([slot], [toks[:head]], [list(range(head))]).cpu()]
        for t in toks[head:]:
            rows.append(engine.step([slot], [[t]], [[0]]).cpu())
        engine.close_sequence(slot)
        out[rid] = torch.cat(rows, dim=0)
    return out


def batched(engine, batches: List[Dict[str, Sequence[int]]], prompt_lens: Dict[str, int]) -> Dict[str, torch.Tensor]:
    """One batch after another. In a batch all requests start together with their first
    ``prompt_lens[id]`` tokens in one step, then go on by one token each; shorter requests end
    earlier and give their slot back at once, so later batches use the slots again."""
    out = {}
    for batch in batches:
        ids = list(batch)
        slots = {rid: engine.open_sequence() for rid in ids}
        rows = {rid: [] for rid in ids}
        lg = engine.step([slots[r] for r in ids], [batch[r][:prompt_lens[r]] for r in ids],
                         [list(range(prompt_lens[r])) for r in ids]).cpu()
        at = 0
        for r in ids:
            rows[r].append(lg[at:at + prompt_lens[r]])
            at += prompt_lens[r]
        done = {r: prompt_lens[r] for r in ids}
        live = [r for r in ids if done[r] < len(batch[r])]
        for r in ids:
            if r not in live:
                engine.close_sequence(slots[r])
        while live:
            lg = engine.step([slots[r] for r in live], [[batch[r][done[r]]] for r in live], [[0]] * len(live)).cpu()
            for i, r in enumerate(live):
                rows[r].append(lg[i:i + 1])
                done[r] += 1
            for r in [r for r in live if done[r] == len(batch[r])]:
                engine.close_sequence(slots[r])
            live = [r for r in live if done[r] < len(batch[r])]
        for r in ids:
            out[r] = torch.cat(rows[r], dim=0)
    return out


def portions(engine, requests: Dict[str, Sequence[int]], size: int, tail: int = 0) -> Dict[str, torch.Tensor]:
    """Each request alone: its tokens in portions of ``size`` onto the cache the earlier portions left; the last
    ``tail`` tokens one by one."""
    out = {}
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        slot = engine.open_sequence()
        rows = []
        for at in range(0, head, size):
            part = toks[at:min(at + size, head)]
            rows.append(engine.step([slot], [part], [list(range(len(part)))]).cpu())
        for t in toks[head:]:
            rows.append(engine.step([slot], [[t]], [[0]]).cpu())
        engine.close_sequence(slot)
        out[rid] = torch.cat(rows, dim=0)
    return out


def joined(engine, first: Dict[str, Sequence[int]], second: Dict[str, Sequence[int]], prompt_lens: Dict[str, int],
           after: int, portion: int = 0) -> Dict[str, torch.Tensor]:
    """The requests of ``first`` start together and decode; after ``after`` decode steps the requests of ``second``
    join them: their prompts (whole, or in portions of ``portion`` tokens) ride in the same steps as the single
    tokens of the running requests. Requests leave when their tokens are used up."""
    batch = dict(first, **second)
    slots, rows, done = {}, {r: [] for r in batch}, {r: 0 for r in batch}
    live: List[str] = []

    def run(entries):   # entries: (request, number of tokens)
        entries = [(r, n) for r, n in entries if n > 0]
        lg = engine.step([slots[r] for r, _ in entries], [batch[r][done[r]:done[r] + n] for r, n in entries],
                         [list(range(n)) for _, n in entries]).cpu()
        at = 0
        for r, n in entries:
            rows[r].append(lg[at:at + n])
            at += n
            done[r] += n
            if done[r] == len(batch[r]):
                engine.close_sequence(slots.pop(r))
                live.remove(r)

    for r in first:
        slots[r] = engine.open_sequence()
        live.append(r)
    run([(r, prompt_lens[r]) for r in first])
    for _ in range(after):
        if live:
            run([(r, 1) for r in list(live)])
    for r in second:
        slots[r] = engine.open_sequence()
        live.append(r)
    while live:
        entries = []
        for r in list(live):
            if r in second and done[r] < prompt_lens[r]:
                left = prompt_lens[r] - done[r]
                entries.append((r, min(left, portion) if portion else left))
            else:
                entries.append((r, 1))
        run(entries)
    return {r: torch.cat(rows[r], dim=0) for r in batch}


def truncated(engine, requests: Dict[str, Sequence[int]], keep: Dict[str, int]) -> Dict[str, torch.Tensor]:
    """Each request alone and whole; then the sequence is cut back to ``keep[id]`` tokens and the rest is fed
    again in one step: the logits of the second pass are returned for the positions from ``keep[id]`` on, those of
    the first pass before."""
    out = {}
    for rid, toks in requests.items():
        slot = engine.open_sequence()
        first = engine.step([slot], [toks], [list(range(len(toks)))]).cpu()
        k = keep[rid]
        engine.cache.truncate(slot, k)
        again = engine.step([slot], [toks[k:]], [list(range(len(toks) - k))]).cpu()
        engine.close_sequence(slot)
        out[rid] = torch.cat([first[:k], again], dim=0)
    return out
