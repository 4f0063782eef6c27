"""The engine on the GPU against the plain implementation, in 32-bit and in bfloat16,
under every way of cutting the same requests: each alone and whole; most of it in one
step and the last 32 tokens one by one; portions of changing size down to two tokens;
and up to four live requests mixed, with so few pages that they are used again.  The
same traces also go through ``bin/trace_run`` as a separate process."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import replay_cases as rc
from tiny_configs import ALL, PAGE_SIZES

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
LENGTHS = {"tiny_a": [5, 11, 17, 40, 23, 64, 100], "tiny_b": [1, 9, 23, 40, 70, 33, 130],
           "tiny_c": [3, 48, 90, 61, 35, 77, 200], "tiny_d": [2, 70, 141, 64, 33, 90, 260]}
# Largest |logit difference| allowed, as a fraction of the largest |logit| of the model.
TOL = {torch.float32: 3e-5, torch.bfloat16: 1.5e-2}


def _oracle(model_dir, reqs):
    cfg, w = plain.read_model_dir(model_dir)
    return {rid: plain.forward_logits(cfg, w, toks, torch.float64).numpy() for rid, toks in reqs}


def _replay(model_dir, name, dtype, steps, page_size=None):
    from emberserve_b200.engine.replay import TraceReplayer
    from emberserve_b200.engine.runner import ModelRunner

    ps = page_size or PAGE_SIZES[name]
    pages = TraceReplayer.pages_for(rc.max_live_tokens(steps), ps)
    runner = ModelRunner.from_dir(model_dir, dtype, page_size=ps, num_pages=pages)
    rp = TraceReplayer(runner)
    outs = {}
    for s in steps:
        o = rp.run_step(s)
        if o is not None:
            outs[s["step"]] = o
        runner.cache.check()
    st = runner.cache.stats()
    assert st.num_sequences == 0 and st.num_free == st.num_pages
    return rc.collect(steps, outs)


def _worst(got, want, reqs):
    worst, where = 0.0, None
    for rid, toks in reqs:
        for p in range(len(toks)):
            e = float(np.abs(got[(rid, p)] - want[rid][p]).max())
            if e > worst:
                worst, where = e, (rid, p)
    return worst, where


@pytest.fixture(scope="module")
def cases(model_dirs):
    out = {}
    for name in ALL:
        reqs = rc.make_requests(ALL[name].vocab_size, LENGTHS[name], seed=7)
        want = _oracle(model_dirs[name], reqs)
        scale = max(float(np.abs(v).max()) for v in want.values())
        out[name] = (reqs, want, scale)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d"])
def test_cut_equals_plain(model_dirs, cases, name, cut, dtype):
    reqs, want, scale = cases[name]
    steps = {"whole": rc.whole, "tail": lambda r: rc.bulk_then_tail(r, 32), "portions": rc.portions,
             "mixed": lambda r: rc.mixed(r, seed=3)}[cut](reqs)
    if cut == "mixed":
        total = sum(-(-len(t) // 64) * 64 for _, t in reqs)
        assert rc.max_live_tokens(steps) < total, "the mixed trace must reuse pages"
    got = _replay(model_dirs[name], name, dtype, steps)
    assert len(got) == sum(len(t) for _, t in reqs)
    worst, where = _worst(got, want, reqs)
    assert worst <= TOL[dtype] * scale, (
        f"{name} {cut} {dtype}: max |dlogit| {worst:.3e} at {where} (logit scale {scale:.3f}, "
        f"allowed {TOL[dtype] * scale:.3e})")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_cuts_agree_with_each_other(model_dirs, cases, dtype):
    """Beyond agreeing with the oracle, the cuts agree with each other much more closely
    in 32-bit: the same kernels see the same numbers in another batch."""
    name = "tiny_b"
    reqs, want, scale = cases[name]
    a = _replay(model_dirs[name], name, dtype, rc.whole(reqs))
    b = _replay(model_dirs[name], name, dtype, rc.mixed(reqs, seed=9))
    worst = max(float(np.abs(a[k] - b[k]).max()) for k in a)
    assert worst <= TOL[dtype] * scale


def test_page_size_16_and_engine_default(model_dirs, cases):
    """The page size the replay program uses (16), not only the tiny ones."""
    name = "tiny_c"
    reqs, want, scale = cases[name]
    got = _replay(model_dirs[name], name, torch.float32, rc.mixed(reqs, seed=1), page_size=16)
    worst, where = _worst(got, want, reqs)
    assert worst <= TOL[torch.float32] * scale, (worst, where)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,block_size", [("tiny_b", None), ("tiny_a", 4)])
def test_trace_run_program(model_dirs, cases, tmp_path, dtype, name, block_size):
    """bin/trace_run as a user runs it: steps on standard input, `done <step>` lines and
    .f32 files back; with its own page size of 16, and with Tiny A's pages of 4 tokens."""
    reqs, want, scale = cases[name]
    steps = rc.mixed(reqs, seed=4)
    out_dir = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dirs[name]), "--dtype", dtype,
         "--out", str(out_dir), "--max-tokens", str(rc.max_live_tokens(steps))]
        + (["--block-size", str(block_size)] if block_size else []),
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    vocab = ALL[name].vocab_size
    outs = {}
    for s in steps:
        f = out_dir / f"{s['step']}.f32"
        if any(e["want"] for e in s["entries"]):
            outs[s["step"]] = np.fromfile(f, dtype="<f4").reshape(-1, vocab)
        else:
            assert not f.exists()
    got = rc.collect(steps, outs)
    worst, where = _worst(got, want, reqs)
    t = TOL[torch.float32 if dtype == "float32" else torch.bfloat16]
    assert worst <= t * scale, (worst, where)
