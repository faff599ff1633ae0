"""Traces for the replay tests: the same requests fed whole, with the tail
decoded one by one, in portions of changing size, and mixed with each other.

A trace is a list of step records in the format of bin/trace_run.  `expected`
maps (request, position) -> the trace step and row that hold its logits, so
that every schedule can be compared with the plain implementation position by
position.
"""

from __future__ import annotations

import numpy as np

PORTIONS = (7, 16, 2, 33, 5, 3, 64, 2, 9, 31, 2, 17)


def _round64(n: int) -> int:
    return -(-n // 64) * 64


def whole(requests: dict[str, list[int]]):
    """Each request alone, its whole token string in one step, logits everywhere."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps, max(_round64(len(t)) for t in requests.values())


def tail(requests: dict[str, list[int]], last: int = 32):
    """All but the last `last` tokens in one step, then one token per step."""
    steps = []
    for rid, toks in requests.items():
        cut = max(1, len(toks) - last)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:cut], "want": list(range(cut))}],
                      "end": []})
        for i in range(cut, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
        if cut == len(toks):
            steps[-1]["end"] = [rid]
    return steps, max(_round64(len(t)) for t in requests.values())


def portions(requests: dict[str, list[int]], sizes=PORTIONS):
    """Each request alone, cut into portions of changing size, down to two tokens."""
    steps = []
    for r, (rid, toks) in enumerate(requests.items()):
        i, k = 0, r
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[i:i + n], "want": list(range(n))}],
                          "end": [rid] if i + n == len(toks) else []})
            i += n
    return steps, max(_round64(len(t)) for t in requests.values())


def mixed(requests: dict[str, list[int]], live: int = 4, seed: int = 0, prompt_fraction: float = 0.6,
          choices=(2, 3, 5, 8, 13, 16, 21, 40)):
    """Up to `live` requests at a time: portions of some beside single decoded
    tokens of others in the same step; a request may sit a step out; requests
    start and end mid-trace, and the pool is so small that pages of finished
    requests are handed to later ones.  Returns (steps, max_tokens)."""
    rng = np.random.default_rng(seed)
    pending = list(requests.items())
    active: dict[str, dict] = {}
    steps = []
    peak = 0
    while pending or active:
        while pending and len(active) < live:
            rid, toks = pending.pop(0)
            active[rid] = {"toks": toks, "done": 0, "prompt": max(1, int(len(toks) * prompt_fraction))}
        entries, ended = [], []
        for rid, st in list(active.items()):
            if len(active) > 1 and rng.random() < 0.15:
                continue                                  # sits this step out
            left = len(st["toks"]) - st["done"]
            if st["done"] < st["prompt"]:
                n = int(min(st["prompt"] - st["done"], rng.choice(list(choices))))
            else:
                n = 1
            n = min(n, left)
            entries.append({"id": rid, "tokens": st["toks"][st["done"]:st["done"] + n], "want": list(range(n))})
            st["done"] += n
            if st["done"] == len(st["toks"]):
                ended.append(rid)
        if not entries:
            continue
        peak = max(peak, sum(_round64(st["done"]) for st in active.values()))
        for rid in ended:
            del active[rid]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps, peak


def keep_wanted(steps, keep) -> list[dict]:
    """The same trace with logits asked for only at the positions `keep(request, position)`
    allows (wide models: a row of logits is large)."""
    at: dict[str, int] = {}
    out = []
    for rec in steps:
        entries = []
        for e in rec["entries"]:
            p0 = at.get(e["id"], 0)
            entries.append({**e, "want": [w for w in e["want"] if keep(e["id"], p0 + w)]})
            at[e["id"]] = p0 + len(e["tokens"])
        out.append({**rec, "entries": entries})
    return out


def wanted_positions(steps) -> dict[str, list[int]]:
    """Per request, the positions whose logits the trace asks for, in the order `collect` returns them."""
    at: dict[str, int] = {}
    pos: dict[str, list[int]] = {}
    for rec in steps:
        for e in rec["entries"]:
            p0 = at.get(e["id"], 0)
            pos.setdefault(e["id"], []).extend(p0 + w for w in e["want"])
            at[e["id"]] = p0 + len(e["tokens"])
    return pos


def collect(steps, outputs: dict[int, np.ndarray]) -> dict[str, np.ndarray]:
    """Per request, the logits of all its positions in order, from the step
    outputs (`outputs[step]` = [wanted, vocab])."""
    rows: dict[str, list[np.ndarray]] = {}
    for rec in steps:
        out = outputs.get(rec["step"])
        r = 0
        for e in rec["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(out[r])
                r += 1
    return {rid: np.stack(v) for rid, v in rows.items()}
