"""Ways of cutting the same requests into steps, in the trace format of bin/trace_run.

Every scenario asks for the logits at every position, so that ``collect`` can put each
request's rows back together as [T, V] and compare them with the plain implementation.
"""
from __future__ import annotations

import random
from typing import Dict, List, Sequence

import torch


def make_requests(lens: Sequence[int], vocab: int, seed: int) -> Dict[str, List[int]]:
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lens)}


def _entry(rid, toks):
    return {"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}


def whole(reqs) -> List[dict]:
    """Each request alone and whole, one step each."""
    return [{"entries": [_entry(r, t)], "end": [r]} for r, t in reqs.items()]


def tail_decode(reqs, tail: int = 32) -> List[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for r, t in reqs.items():
        head = max(1, len(t) - tail)
        steps.append({"entries": [_entry(r, t[:head])], "end": []})
        for i in range(head, len(t)):
            steps.append({"entries": [_entry(r, t[i:i + 1])], "end": []})
        steps[-1]["end"] = [r]
    return steps


def portions(reqs, seed: int = 0) -> List[dict]:
    """Portions of changing size, down to two tokens and one."""
    rng = random.Random(seed)
    steps = []
    for r, t in reqs.items():
        i = 0
        sizes = [2, 1, 3, 2, 17, 2, 5, 31, 2, 64, 7]
        k = 0
        while i < len(t):
            n = min(len(t) - i, sizes[k % len(sizes)] if k < 2 * len(sizes) else rng.choice(sizes))
            steps.append({"entries": [_entry(r, t[i:i + n])], "end": []})
            i += n
            k += 1
        steps[-1]["end"] = [r]
    return steps


def mixed(reqs, capacity_tokens: int, round_to: int = 64, seed: int = 0, max_live: int = 4) -> List[dict]:
    """Up to ``max_live`` live requests: portions of some beside single decode tokens of
    others.  A request is admitted only if, with every live request's final length rounded up
    to ``round_to``, all fit in ``capacity_tokens``; so pages given back are used again."""
    rng = random.Random(seed)
    up = lambda n: -(-n // round_to) * round_to
    waiting, live, fed = list(reqs), [], {r: 0 for r in reqs}
    prefill_until = {r: max(1, len(t) - rng.choice([0, 8, 32])) for r, t in reqs.items()}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and \
                sum(up(len(reqs[r])) for r in live) + up(len(reqs[waiting[0]])) <= capacity_tokens:
            live.append(waiting.pop(0))
        assert live, "capacity too small for the next request"
        entries, end = [], []
        for r in live:
            t = reqs[r]
            if fed[r] < prefill_until[r]:
                n = min(prefill_until[r] - fed[r], rng.choice([2, 3, 16, 16, 40]))
            else:
                n = 1
            if rng.random() < 0.15 and len(live) > 1:
                continue                                   # a request may sit out a step
            entries.append(_entry(r, t[fed[r]:fed[r] + n]))
            fed[r] += n
            if fed[r] == len(t):
                end.append(r)
        if not entries:
            continue
        steps.append({"entries": entries, "end": end})
        for r in end:
            live.remove(r)
    return steps


def number(steps: List[dict]) -> List[dict]:
    return [dict(s, step=i) for i, s in enumerate(steps)]


def collect(steps: List[dict], logits_of_step) -> Dict[str, torch.Tensor]:
    """``logits_of_step(i)`` -> tensor [wanted, V] of step i.  Returns request -> [T, V]."""
    parts: Dict[str, list] = {}
    for i, s in enumerate(steps):
        lg = logits_of_step(i)
        o = 0
        for e in s["entries"]:
            n = len(e["want"])
            parts.setdefault(e["id"], []).append(lg[o:o + n])
            o += n
    return {r: torch.cat(p) for r, p in parts.items()}
