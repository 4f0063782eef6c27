"""Trace replay: feed given token ids through the model step by step and hand back logits.

A trace is a sequence of steps; a step names, for each request in it, its next tokens
and the places among them whose logits are wanted, and the requests that end after it:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

The replayer samples nothing.  It owns no forward pass, cache or loader: it reserves
pages through the runner's cache manager and calls ``ModelRunner.step``, the function
that generation uses.  The reference's nearest tools are ``scripts/dump_golden.py`` and
``scripts/check_golden.py:27-37`` (schedule a whole prompt, read all-position logits);
an explicit per-step schedule is this package's own.
"""

from __future__ import annotations

import numpy as np

from emberserve_b200 import kernels as K
from emberserve_b200.engine.runner import ModelRunner, StepRow


class TraceError(ValueError):
    pass


class TraceReplayer:
    def __init__(self, runner: ModelRunner) -> None:
        self.runner = runner
        self._ids: dict[str, int] = {}
        self._next_seq = 0
        self._length: dict[str, int] = {}

    @staticmethod
    def pages_for(max_tokens: int, page_size: int) -> int:
        """Pages of a pool that must hold `max_tokens` tokens of live requests."""
        return max(1, -(-max_tokens // page_size))

    def run_step(self, step: dict) -> np.ndarray | None:
        """Run one step; returns float32 logits [wanted, vocab] in the order of the entries
        and of their `want`, or None when nothing is wanted."""
        cache = self.runner.cache
        rows: list[StepRow] = []
        for entry in step.get("entries", []):
            rid = str(entry["id"])
            tokens = [int(t) for t in entry["tokens"]]
            if not tokens:
                raise TraceError(f"step {step.get('step')}: request {rid!r} brings no tokens")
            if rid not in self._ids:
                self._ids[rid] = self._next_seq
                self._next_seq += 1
                self._length[rid] = 0
                cache.admit(self._ids[rid], len(tokens))
            else:
                cache.extend(self._ids[rid], self._length[rid] + len(tokens))
            rows.append(StepRow(self._ids[rid], tokens, self._length[rid],
                                [int(w) for w in entry.get("want", [])]))
            self._length[rid] += len(tokens)
        logits = self.runner.step(rows) if rows else None
        out = None
        if logits is not None and logits.shape[0] > 0:
            out = logits.detach().to("cpu").numpy().astype("<f4", copy=True)
            K.check_status()  # the copy waited for the step: no logits of a kernel that gave up
        for rid in step.get("end", []):
            rid = str(rid)
            if rid in self._ids:
                cache.release(self._ids.pop(rid))
                self._length.pop(rid, None)
        return out
