"""The scheduler's decisions, without tensors: a fake loop plays the engine, its "model"
is next = (last * 7 + 3) % 256 (the idea of the reference's tests/fakes.py)."""

from __future__ import annotations

import pytest

from emberserve_b200.cache.manager import CacheManager, plan_groups
from emberserve_b200.config.engine import EngineConfig
from emberserve_b200.engine.request import FinishReason, Request, RequestState, check_stop
from emberserve_b200.engine.scheduler import Scheduler
from emberserve_b200.parts.base import PagedKV
from emberserve_b200.sampling.params import SamplingParams


def next_token(last: int) -> int:
    return (last * 7 + 3) % 256


class FakeLoop:
    def __init__(self, pages=64, page_size=4, **cfg):
        self.cfg = EngineConfig(block_size=page_size, **cfg)
        self.cache = CacheManager(plan_groups([PagedKV(1, 16, None)]), pages, page_size)
        self.sched = Scheduler(self.cfg, self.cache)
        self.n = 0
        self.log = []  # per step: list of (request_id, query_len, complete)
        self.preemptions = []

    def add(self, rid, prompt, max_tokens=4, **kw):
        req = Request(rid, list(prompt), SamplingParams.greedy(max_tokens, **kw), seq_id=self.n)
        self.n += 1
        self.sched.add_request(req)
        return req

    def step(self):
        so = self.sched.schedule()
        self.preemptions += [r.request_id for r in so.preempted]
        if so.is_empty:
            return so
        assert len({id(r) for r in so.scheduled}) == len(so.scheduled)
        self.log.append([(r.request_id, q, c) for r, q, c in zip(so.scheduled, so.query_lens, so.prefill_complete)])
        for req, q, done in zip(so.scheduled, so.query_lens, so.prefill_complete):
            assert 1 <= q and req.num_computed_tokens + q <= self.cache.num_tokens(req.seq_id)
            self.cache.commit(req.seq_id, req.num_computed_tokens + q)
            req.num_computed_tokens += q
            assert done == (req.num_computed_tokens == req.num_tokens)
            if done:
                tok = next_token(req.all_token_ids[-1])
                req.append_output(tok)
                reason = check_stop(req, tok, frozenset({1}), self.cfg.max_model_len)
                if reason is not None:
                    self.sched.finish_request(req, reason)
        self.cache.check()
        return so

    def run(self, limit=1000):
        for _ in range(limit):
            if not self.sched.has_unfinished_requests():
                return
            self.step()
        raise AssertionError("the loop did not finish")


def expected(prompt, n):
    out, last = [], prompt[-1]
    for _ in range(n):
        last = next_token(last)
        out.append(last)
    return out


def test_rejections():
    loop = FakeLoop(max_model_len=16, max_num_batched_tokens=8, enable_chunked_prefill=False)
    with pytest.raises(ValueError, match="empty"):
        loop.add("a", [])
    with pytest.raises(ValueError, match="max_model_len"):
        loop.add("b", [5] * 16)
    with pytest.raises(ValueError, match="max_num_batched_tokens"):
        loop.add("c", [5] * 9)
    loop.add("d", [5] * 8)
    with pytest.raises(ValueError, match="duplicate"):
        loop.add("d", [5])
    chunked = FakeLoop(max_model_len=16, max_num_batched_tokens=8)
    chunked.add("c", [5] * 9)  # a long prompt is simply cut into portions


def test_fifo_never_skips_ahead():
    loop = FakeLoop(pages=6, page_size=4, enable_chunked_prefill=False)
    loop.add("big", [9] * 20)  # 5 pages (+1 for its first token)
    loop.add("huge", [9] * 23)  # does not fit beside it
    loop.add("small", [9] * 2)  # would fit, but stands behind `huge`
    loop.step()
    assert [r for r, _, _ in loop.log[0]] == ["big"]
    loop.step()
    assert [r for r, _, _ in loop.log[1]] == ["big"] and loop.sched.num_waiting == 2


def test_max_num_seqs_and_budget_unchunked():
    loop = FakeLoop(max_num_seqs=2, max_num_batched_tokens=10, enable_chunked_prefill=False)
    for i in range(4):
        loop.add(f"r{i}", [3] * 6, max_tokens=2)
    loop.step()
    assert loop.log[0] == [("r0", 6, True)]  # 6 + 6 > 10: one prompt per step
    loop.step()
    assert loop.log[1] == [("r1", 6, True)]
    loop.step()  # two are running: a decode step, nobody new
    assert loop.log[2] == [("r0", 1, True), ("r1", 1, True)]
    loop.run()
    assert all(len(s) <= 2 for s in loop.log)


def test_chunked_splits_prompt_and_keeps_decodes_flowing():
    loop = FakeLoop(max_num_batched_tokens=32, pages=128)
    a = loop.add("a", [4] * 3, max_tokens=50)
    loop.step()
    b = loop.add("b", [5] * 100, max_tokens=3)
    chunks = []
    while b.num_computed_tokens < 100:
        so = loop.step()
        assert so.num_tokens <= 32
        rows = dict((r, (q, c)) for r, q, c in loop.log[-1])
        assert rows["a"] == (1, True)  # the decoding request gets its token in every step
        assert loop.log[-1][0][0] == "a"  # decode rows come first
        chunks.append(rows["b"][0])
        assert rows["b"][1] == (sum(chunks) == 100)
    assert chunks == [31, 31, 31, 7]
    loop.run()
    assert a.output_token_ids == expected([4] * 3, 50) and b.output_token_ids == expected([5] * 100, 3)


def test_chunked_oldest_mid_prompt_first_then_new():
    loop = FakeLoop(max_num_batched_tokens=10, pages=128)
    loop.add("a", [1 + i for i in range(14)])
    loop.add("b", [2] * 8)
    loop.step()
    assert loop.log[0] == [("a", 10, False)]
    loop.step()
    assert loop.log[1] == [("a", 4, True), ("b", 6, False)]
    loop.step()
    assert loop.log[2] == [("a", 1, True), ("b", 2, True)]


@pytest.mark.parametrize("chunked", [False, True])
def test_pages_run_out_youngest_is_preempted_and_outputs_survive(chunked):
    loop = FakeLoop(pages=10, page_size=4, enable_chunked_prefill=chunked, max_num_batched_tokens=64)
    reqs = [loop.add(f"r{i}", [10 + i] * 7, max_tokens=20) for i in range(3)]
    loop.run()
    assert loop.preemptions, "the pool was chosen too small for three requests to finish together"
    assert loop.preemptions[0] == "r2"  # the youngest goes first
    for i, r in enumerate(reqs):
        assert r.output_token_ids == expected([10 + i] * 7, 20) and r.finish_reason == FinishReason.LENGTH
    assert loop.cache.stats().num_free == loop.cache.stats().num_pages


def test_preempted_request_returns_to_the_front_and_recomputes_everything():
    loop = FakeLoop(pages=10, page_size=4, max_num_batched_tokens=64)
    a = loop.add("a", [3] * 8, max_tokens=30)
    b = loop.add("b", [4] * 8, max_tokens=30)
    while not loop.preemptions:
        loop.step()
    assert loop.preemptions == ["b"] and b.state == RequestState.PREEMPTED
    assert loop.sched.waiting[0] is b and b.num_computed_tokens == 0 and b.num_output_tokens > 0
    kept = list(b.output_token_ids)
    loop.run()
    assert b.output_token_ids[:len(kept)] == kept and b.output_token_ids == expected([4] * 8, 30)
    assert a.output_token_ids == expected([3] * 8, 30)
    # its recomputation covered prompt + kept outputs
    redo = [q for s in loop.log for r, q, _ in s if r == "b" and q > 1]
    assert sum(redo) >= 8 + 8 + len(kept) - 1


def test_lone_request_that_cannot_grow_waits_instead_of_looping():
    loop = FakeLoop(pages=2, page_size=4, max_model_len=64)
    r = loop.add("a", [3] * 7, max_tokens=30)
    for _ in range(40):
        loop.step()
    # 8 slots: prompt 7 + 1 decode fits, then it preempts itself and can never be re-admitted
    assert r.num_output_tokens >= 2 and not r.is_finished
    loop.sched.abort_request("a")
    assert r.finish_reason == FinishReason.ABORT and loop.cache.stats().num_free == [2]


def test_abort_in_every_state_and_stop_rules():
    loop = FakeLoop(max_num_seqs=1)
    a = loop.add("a", [3] * 5, max_tokens=9)
    b = loop.add("b", [4] * 5)
    loop.step()
    loop.sched.abort_request("b")  # waiting
    loop.sched.abort_request("a")  # running
    assert a.finish_reason == b.finish_reason == FinishReason.ABORT
    assert loop.sched.abort_request("zzz") is None and not loop.sched.has_unfinished_requests()
    assert loop.cache.stats().num_sequences == 0
    r = Request("x", [1, 2], SamplingParams.greedy(2, stop_token_ids=[9]))
    r.append_output(9)
    assert check_stop(r, 9, frozenset({1}), 100) == FinishReason.STOP
    r.append_output(1)
    assert check_stop(r, 1, frozenset({1}), 100) == FinishReason.STOP  # STOP wins over LENGTH
    r.sampling_params.ignore_eos = True
    assert check_stop(r, 1, frozenset({1}), 100) == FinishReason.LENGTH
    r2 = Request("y", [1, 2, 3], SamplingParams.greedy(50))
    r2.append_output(5)
    assert check_stop(r2, 5, frozenset({1}), 4) == FinishReason.LENGTH  # model length
    assert check_stop(r2, 5, frozenset({1}), 5) is None
