"""Traces for the replay tests: the same requests cut in four ways.

A trace is a list of step dicts in the format of ``bin/trace_run``.  Every cut asks for
the logits of every position of every request, so that all cuts can be compared with the
plain implementation position by position (``collect`` sorts what came back).
"""

from __future__ import annotations

import random

import numpy as np

Request = tuple[str, list[int]]  # (id, all its token ids)


def make_requests(vocab: int, lengths: list[int], seed: int) -> list[Request]:
    rng = random.Random(seed)
    return [(f"r{i}", [rng.randrange(vocab) for _ in range(n)]) for i, n in enumerate(lengths)]


def whole(reqs: list[Request]) -> list[dict]:
    """Each request alone and whole: one step with all its tokens."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
             "end": [rid]} for i, (rid, toks) in enumerate(reqs)]


def bulk_then_tail(reqs: list[Request], tail: int = 32) -> list[dict]:
    """Most of a request in one step, the last `tail` tokens one by one.  A request no
    longer than the tail starts with a one-token step."""
    steps: list[dict] = []
    for rid, toks in reqs:
        bulk = max(1, len(toks) - tail)
        steps.append({"entries": [{"id": rid, "tokens": toks[:bulk], "want": list(range(bulk))}], "end": []})
        for p in range(bulk, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return _number(steps)


def portions(reqs: list[Request], sizes: tuple[int, ...] = (7, 5, 3, 2, 11, 2, 4, 9, 2, 6)) -> list[dict]:
    """Portions of changing size, down to two tokens, never the same size twice in a row."""
    steps: list[dict] = []
    for r, (rid, toks) in enumerate(reqs):
        p, k = 0, r  # each request starts at another place of the size pattern
        while p < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            steps.append({"entries": [{"id": rid, "tokens": toks[p:p + n], "want": list(range(n))}], "end": []})
            p += n
        steps[-1]["end"] = [rid]
    return _number(steps)


def mixed(reqs: list[Request], max_live: int = 4, seed: int = 0, decode_tail: int = 12,
          chunk_sizes: tuple[int, ...] = (5, 2, 9, 3, 7, 2, 13)) -> list[dict]:
    """Up to `max_live` live requests: portions of some beside single tokens of others in
    the same step, arrivals staggered, some requests skipped in some steps.  A request's
    last `decode_tail` tokens come one per step (decoding).  Requests end as soon as they
    are done, so that with a small pool their pages go to the requests that follow."""
    rng = random.Random(seed)
    waiting = list(reqs)
    live: list[dict] = []
    steps: list[dict] = []
    while waiting or live:
        # admit at most one new request per step, so that arrivals are staggered
        if waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live.append({"id": rid, "toks": toks, "pos": 0, "k": rng.randrange(len(chunk_sizes))})
        entries, ended = [], []
        for st in live:
            if len(live) > 1 and rng.random() < 0.2 and st["pos"] > 0:
                continue  # left out of this step, goes on later
            left = len(st["toks"]) - st["pos"]
            if left <= decode_tail and st["pos"] > 0:
                n = 1
            else:
                n = min(chunk_sizes[st["k"] % len(chunk_sizes)], max(1, left - decode_tail))
                st["k"] += 1
            entries.append({"id": st["id"], "tokens": st["toks"][st["pos"]:st["pos"] + n],
                            "want": list(range(n))})
            st["pos"] += n
            if st["pos"] == len(st["toks"]):
                ended.append(st["id"])
        live = [st for st in live if st["id"] not in ended]
        if entries:
            steps.append({"entries": entries, "end": ended})
    return _number(steps)


def _number(steps: list[dict]) -> list[dict]:
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def max_live_tokens(steps: list[dict], round_to: int = 64) -> int:
    """The most tokens that live requests hold at any time, each request's count rounded
    up to a multiple of `round_to` (what ``--max-tokens`` has to cover)."""
    length: dict[str, int] = {}
    worst = 0
    for s in steps:
        for e in s["entries"]:
            length[e["id"]] = length.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // round_to) * round_to for n in length.values()))
        for rid in s["end"]:
            length.pop(rid, None)
    return worst


def collect(steps: list[dict], outputs: dict[int, np.ndarray]) -> dict[tuple[str, int], np.ndarray]:
    """(request id, position) -> logits row, from the per-step arrays."""
    pos: dict[str, int] = {}
    got: dict[tuple[str, int], np.ndarray] = {}
    for s in steps:
        row = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = outputs[s["step"]][row]
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            pos.pop(rid, None)
        if s["step"] in outputs:
            assert outputs[s["step"]].shape[0] == row, "the step returned another number of rows"
    return got
