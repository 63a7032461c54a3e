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
