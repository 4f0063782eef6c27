"""The step function, the cache and the replay driver against the plain implementation,
on the CPU with the kernels' restatements (see host_harness.py): every way of cutting
the same requests gives the same logits."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import kernel_refs
import plain_qwen2 as plain
import replay_cases as rc
from host_harness import host_runner
from tiny_configs import ALL, PAGE_SIZES

from emberserve_b200.engine.replay import TraceReplayer

LENGTHS = {"tiny_a": [5, 11, 17, 40, 23, 64], "tiny_b": [1, 9, 23, 40, 70, 33],
           "tiny_c": [3, 48, 90, 61, 35, 77], "tiny_d": [2, 70, 141, 64, 33, 90]}


@pytest.fixture(autouse=True)
def _refs(monkeypatch):
    kernel_refs.install(monkeypatch)


def _replay(model_dir, name, steps, num_pages=None):
    ps = PAGE_SIZES[name]
    pages = num_pages or TraceReplayer.pages_for(rc.max_live_tokens(steps), ps)
    runner = host_runner(model_dir, page_size=ps, num_pages=pages)
    rp = TraceReplayer(runner)
    outs = {}
    for s in steps:
        o = rp.run_step(s)
        if o is not None:
            outs[s["step"]] = o
        runner.cache.check()
    assert runner.cache.stats().num_sequences == 0
    assert all(f == n for f, n in zip(runner.cache.stats().num_free, runner.cache.stats().num_pages))
    return rc.collect(steps, outs)


def _oracle(model_dir, reqs):
    cfg, w = plain.read_model_dir(model_dir)
    return {rid: plain.forward_logits(cfg, w, toks, torch.float64).numpy() for rid, toks in reqs}


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d"])
def test_all_cuts_equal_plain(model_dirs, name):
    cfg = ALL[name]
    reqs = rc.make_requests(cfg.vocab_size, LENGTHS[name], seed=7)
    want = _oracle(model_dirs[name], reqs)
    scale = max(float(np.abs(v).max()) for v in want.values())
    cuts = {"whole": rc.whole(reqs), "tail": rc.bulk_then_tail(reqs, 32),
            "portions": rc.portions(reqs), "mixed": rc.mixed(reqs, seed=3)}
    for cut, steps in cuts.items():
        got = _replay(model_dirs[name], name, steps)
        assert len(got) == sum(len(t) for _, t in reqs), cut
        worst = max(float(np.abs(got[(rid, p)] - want[rid][p]).max())
                    for rid, toks in reqs for p in range(len(toks)))
        assert worst <= 2e-5 * scale, f"{name} {cut}: max |dlogit| {worst:.3e} (scale {scale:.3f})"


def test_mixed_reuses_pages(model_dirs):
    name = "tiny_a"
    reqs = rc.make_requests(ALL[name].vocab_size, LENGTHS[name], seed=11)
    steps = rc.mixed(reqs, seed=5)
    need = rc.max_live_tokens(steps)
    total = sum(-(-len(t) // 64) * 64 for _, t in reqs)
    assert need < total, "the trace must not fit without giving pages back"
    got = _replay(model_dirs[name], name, steps)
    want = _oracle(model_dirs[name], reqs)
    for rid, toks in reqs:
        for p in range(len(toks)):
            assert np.abs(got[(rid, p)] - want[rid][p]).max() < 1e-4
