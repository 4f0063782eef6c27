"""The engine on the GPU beyond the four cuts: greedy generation through the entry point,
long decoding, the first tokens of a sequence, faults that random weights would hide
(a far key, a window's edge, a page's edge), each part alone, and a toy architecture with
a mixer that has state of its own, registered from here without touching the package."""

from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass
from typing import ClassVar

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import replay_cases as rc
from tiny_configs import ALL, PAGE_SIZES, SEEDS

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
# Largest |logit difference| allowed, as a fraction of the model's largest |logit|: with the
# ordinary random weights N(0, 0.02) (bfloat16 measured at 5e-3), and with the "sharp" weights of
# five times the deviation or scaled q/k projections, whose logits bfloat16 rounding moves more.
TOL = {torch.float32: 3e-5, torch.bfloat16: 1.5e-2}
TOL_SHARP = {torch.float32: 3e-5, torch.bfloat16: 3e-2}


def _runner(model_dir, dtype, page_size, pages):
    from emberserve_b200.engine.runner import ModelRunner

    return ModelRunner.from_dir(model_dir, dtype, device=DEV, page_size=page_size, num_pages=pages)


def _llm(model_dir, name, dtype, pages=512, **cfg):
    from emberserve_b200 import LLM

    return LLM(model_dir, dtype=dtype, device=DEV, block_size=PAGE_SIZES[name], num_gpu_blocks=pages,
               max_model_len=ALL[name].max_position_embeddings, **cfg)


def _sharp_model(tmp_path_factory, name, std=0.1):
    """Weights with five times the usual deviation: logits far enough apart that greedy
    tokens vary and mean something, while the model stays well conditioned (ten times the
    deviation makes these tiny models chaotic: bfloat16 rounding alone then moves logits by
    several per cent)."""
    from emberserve_b200.weights.loader import write_random_model

    return write_random_model(ALL[name], tmp_path_factory.mktemp(f"sharp_{name}"), SEEDS[name], std=std,
                              bias_std=std)


@pytest.fixture(scope="module")
def sharp_dirs(tmp_path_factory):
    return {name: _sharp_model(tmp_path_factory, name) for name in ALL}


# ---- generation through the entry point ---------------------------------------------------------

@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d"])
def test_greedy_generation_equals_plain(sharp_dirs, name):
    from emberserve_b200 import SamplingParams

    cfg, w = plain.read_model_dir(sharp_dirs[name])
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, ALL[name].vocab_size, (n,), generator=g).tolist() for n in (5, 11, 17)]
    want = [plain.greedy_generate(cfg, w, p, 8) for p in prompts]
    llm = _llm(sharp_dirs[name], name, "float32")
    got = [r.output_token_ids for r in llm.generate(prompts, SamplingParams.greedy(8, ignore_eos=True))]
    assert got == want
    # bfloat16: a token may differ only where the plain logits of the two candidates are
    # closer than the bfloat16 error of the engine (the reference's rule,
    # scripts/check_golden.py:55-117)
    got16 = [r.output_token_ids for r in
             _llm(sharp_dirs[name], name, "bfloat16").generate(prompts, SamplingParams.greedy(8, ignore_eos=True))]
    for p, a, b in zip(prompts, got16, want):
        for i, (x, y) in enumerate(zip(a, b)):
            if x != y:
                logits = plain.forward_logits(cfg, w, p + b[:i])[-1]
                assert abs(float(logits[x] - logits[y])) <= 2 * TOL_SHARP[torch.bfloat16] * float(logits.abs().max())
                break


def test_chunked_mixed_and_preempted_generation_on_the_gpu(sharp_dirs):
    from emberserve_b200 import SamplingParams

    name = "tiny_b"
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, ALL[name].vocab_size, (n,), generator=g).tolist() for n in (1, 9, 23, 40)]
    params = [SamplingParams(max_tokens=12, temperature=0.8, seed=7 + i, ignore_eos=True) for i in range(4)]
    base = [r.output_token_ids for r in _llm(sharp_dirs[name], name, "float32",
                                             enable_chunked_prefill=False).generate(prompts, params)]
    llm = _llm(sharp_dirs[name], name, "float32", max_num_batched_tokens=7)
    llm.engine.keep_stats = True
    assert [r.output_token_ids for r in llm.generate(prompts, params)] == base
    assert any(s.num_decode_tokens and s.num_prefill_tokens for s in llm.engine.stats)
    tight = _llm(sharp_dirs[name], name, "float32", pages=13, max_num_batched_tokens=16)
    tight.engine.keep_stats = True
    assert [r.output_token_ids for r in tight.generate(prompts, params)] == base
    assert sum(s.num_preempted for s in tight.engine.stats) >= 1
    st = tight.engine.runner.cache.stats()
    assert st.num_free == st.num_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", [dict(), dict(max_num_batched_tokens=8), dict(pages=6, max_num_batched_tokens=64)])
def test_async_scheduling_changes_no_token_on_the_gpu(sharp_dirs, dtype, how):
    """Steps launched before the tokens of the step before them are read (the sampled tokens
    feed the next step on the device, decode steps replay CUDA graphs) give the tokens and
    finish reasons of plain stepping: requests ending by an end-of-sequence token, a stop
    token, max_tokens and the model length, sampled and greedy, chunked and preempted."""
    from emberserve_b200 import SamplingParams
    from emberserve_b200.engine.request import FinishReason

    name = "tiny_b"
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, ALL[name].vocab_size, (n,), generator=g).tolist() for n in (7, 19, 3, 26, 11, 15)]
    probe = _llm(sharp_dirs[name], name, dtype, async_scheduling=False)
    free = probe.generate(prompts[:2], SamplingParams.greedy(10, ignore_eos=True))
    params = [
        SamplingParams.greedy(10, stop_token_ids=[free[0].output_token_ids[3]], ignore_eos=True),
        SamplingParams.greedy(10),
        SamplingParams(max_tokens=9, temperature=0.9, seed=5, ignore_eos=True),
        SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True),
        SamplingParams(max_tokens=14, temperature=0.6, top_k=7, seed=6, ignore_eos=True),
        SamplingParams(max_tokens=60, temperature=0.0, ignore_eos=True),
    ]
    eos = frozenset({free[1].output_token_ids[5]})
    results = []
    for async_on in (False, True):
        llm = _llm(sharp_dirs[name], name, dtype, async_scheduling=async_on, **how)
        llm.engine.config.max_model_len = 40
        llm.engine.eos_token_ids = eos
        llm.engine.keep_stats = True
        res = llm.generate(prompts, params)
        results.append([(r.output_token_ids, r.finish_reason) for r in res])
        st = llm.engine.runner.cache.stats()
        assert st.num_free == st.num_pages and st.num_sequences == 0
        assert all(0 <= t < ALL[name].vocab_size for r in res for t in r.output_token_ids)
        if "pages" in how:
            assert sum(s.num_preempted for s in llm.engine.stats) >= 1, "the pool was not tight enough"
    assert results[0] == results[1]
    assert [r for _, r in results[0]][:2] == [FinishReason.STOP, FinishReason.STOP]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_d"])
def test_no_kernel_writes_outside_its_scratch_buffers(sharp_dirs, name, dtype):
    """Generation with guard elements around every scratch buffer of the steps (eager and graph
    arenas): whole prompts, portions, decode steps from graphs, sampled and greedy.  The engine
    checks the guards after every step and raises if a kernel wrote there."""
    from emberserve_b200 import SamplingParams

    g = torch.Generator().manual_seed(5)
    top = min(100, ALL[name].max_position_embeddings - 20)
    prompts = [torch.randint(0, ALL[name].vocab_size, (n,), generator=g).tolist() for n in (1, 9, 33, top, 70)]
    params = [SamplingParams.greedy(8, ignore_eos=True), SamplingParams(max_tokens=8, temperature=0.8, seed=1, ignore_eos=True),
              SamplingParams(max_tokens=8, temperature=1.0, top_k=5, top_p=0.9, seed=2, ignore_eos=True),
              SamplingParams.greedy(8, ignore_eos=True), SamplingParams.greedy(8, ignore_eos=True)]
    for how in (dict(), dict(max_num_batched_tokens=16), dict(enable_cuda_graphs=False, async_scheduling=False)):
        llm = _llm(sharp_dirs[name], name, dtype, debug_scratch_guard=64, **how)
        assert llm.engine.runner.scratch.guard == 64
        res = llm.generate(prompts, params)
        assert all(len(r.output_token_ids) == 8 for r in res)
        llm.engine.runner.verify_scratch()


@pytest.mark.parametrize("backend", ["auto", "mma", "generic"])
def test_attention_backend_of_the_engine(sharp_dirs, backend, monkeypatch):
    """EngineConfig.attn_backend reaches the kernels (every attention launch of the engine names
    it; the fused decode kernel is not used with "generic") and the logits stay those of the
    plain implementation."""
    from emberserve_b200 import SamplingParams
    from emberserve_b200 import kernels as K

    name = "tiny_d"
    cfg, w = plain.read_model_dir(sharp_dirs[name])
    seen, fused = [], []
    real_paged, real_fused = K.paged_attention, K.decode_attention_fused
    monkeypatch.setattr(K, "paged_attention", lambda *a, **kw: (seen.append(kw.get("kernel")), real_paged(*a, **kw))[1])
    monkeypatch.setattr(K, "decode_attention_fused", lambda *a, **kw: (fused.append(1), real_fused(*a, **kw))[1])
    llm = _llm(sharp_dirs[name], name, "bfloat16", attn_backend=backend, enable_cuda_graphs=False)
    g = torch.Generator().manual_seed(31)
    prompt = torch.randint(0, ALL[name].vocab_size, (40,), generator=g).tolist()
    res = llm.generate([prompt], SamplingParams.greedy(5, ignore_eos=True))[0]
    assert len(res.output_token_ids) == 5
    assert seen and set(seen) == {backend}
    assert bool(fused) == (backend != "generic")
    eng = llm.engine
    eng.add_request("logits", prompt, SamplingParams.greedy(1))
    logits = eng.step_logits(eng.scheduler.schedule(), all_positions=True).double().cpu()
    eng.abort_request("logits")
    ref = plain.forward_logits(cfg, w, prompt)
    assert float((logits - ref).abs().max()) <= 3e-2 * float(ref.abs().max())
    with pytest.raises(ValueError, match="attn_backend"):
        _llm(sharp_dirs[name], name, "bfloat16", attn_backend="flash")


def test_released_graphs_change_no_token(sharp_dirs):
    """release_graphs() lets go of the captured decode graphs; the engine then launches its kernels
    one by one and generates the same tokens (also with a step still in flight at the release)."""
    from emberserve_b200 import SamplingParams

    name = "tiny_b"
    g = torch.Generator().manual_seed(23)
    prompts = [torch.randint(0, ALL[name].vocab_size, (n,), generator=g).tolist() for n in (9, 4, 13)]
    llm = _llm(sharp_dirs[name], name, "float32", pages=64)
    assert llm.engine.runner.graphs is not None
    want = [r.output_token_ids for r in llm.generate(prompts, SamplingParams.greedy(12, ignore_eos=True))]
    for i, p in enumerate(prompts):
        llm.engine.add_request(f"again-{i}", p, SamplingParams.greedy(12, ignore_eos=True))
    got: dict[str, list[int]] = {}
    steps = 0
    while llm.engine.has_unfinished_requests():
        for out in llm.engine.step():
            if out.finished:
                got[out.request_id] = out.output_token_ids
        steps += 1
        if steps == 5:
            llm.engine.release_graphs()
            assert llm.engine.runner.graphs is None
    assert [got[f"again-{i}"] for i in range(len(prompts))] == want


def test_command_line_generates_what_the_entry_point_generates(sharp_dirs):
    """`python -m emberserve_b200 generate --prompt-ids ...` prints the tokens that
    LLM.generate() returns, and the throughput line on standard error."""
    import subprocess
    import sys
    from pathlib import Path

    from emberserve_b200 import SamplingParams

    name = "tiny_b"
    prompt = [7, 100, 33, 250, 9]
    want = _llm(sharp_dirs[name], name, "float32").generate([prompt], SamplingParams.greedy(6, ignore_eos=True))
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run(
        [sys.executable, "-m", "emberserve_b200", "generate", "--model", str(sharp_dirs[name]), "--dtype",
         "float32", "--block-size", "8", "--num-blocks", "64", "--max-model-len", "200", "--prompt-ids",
         ",".join(map(str, prompt)), "--max-tokens", "6"],
        capture_output=True, text=True, cwd=root, timeout=600)
    assert proc.returncode == 0, proc.stderr[-1500:]
    got = [int(t) for t in proc.stdout.split()]
    # the command line stops at an end-of-sequence token, the call above ignored it
    assert got == want[0].output_token_ids[:len(got)] and 1 <= len(got) <= 6
    assert "tokens in" in proc.stderr and "finish=" in proc.stderr


def test_cpu_device_is_refused(model_dirs):
    from emberserve_b200.engine.runner import ModelRunner

    with pytest.raises(RuntimeError, match="CUDA GPU only"):
        ModelRunner.from_dir(model_dirs["tiny_a"], torch.float32, device="cpu")


# ---- long decoding and the first tokens ---------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_c", "tiny_d"])
def test_long_decoding_token_by_token(sharp_dirs, name, dtype):
    """A short prompt and then every further token alone, across many pages (and, for the
    windowed model, far past the window, while its pages are given back)."""
    from emberserve_b200.engine.replay import TraceReplayer

    cfg = ALL[name]
    n = cfg.max_position_embeddings - 3
    reqs = rc.make_requests(cfg.vocab_size, [n], seed=5)
    cfgd, w = plain.read_model_dir(sharp_dirs[name])
    want = plain.forward_logits(cfgd, w, reqs[0][1]).numpy()
    steps = rc.bulk_then_tail(reqs, tail=n - 3)
    ps = PAGE_SIZES[name]
    runner = _runner(sharp_dirs[name], dtype, ps, -(-n // ps))
    rp = TraceReplayer(runner)
    outs = {s["step"]: rp.run_step(s) for s in steps}
    got = rc.collect(steps, outs)
    err = max(float(np.abs(got[("r0", p)] - want[p]).max()) for p in range(n))
    assert err <= TOL_SHARP[dtype] * float(np.abs(want).max()), err
    if name == "tiny_c":
        assert runner.cache.stats().num_free[1] == runner.cache.stats().num_pages[1]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_first_tokens_of_a_sequence(sharp_dirs, dtype):
    """Sequences of one, two and three tokens, token by token and whole, beside each other."""
    from emberserve_b200.engine.replay import TraceReplayer

    name = "tiny_b"
    reqs = rc.make_requests(ALL[name].vocab_size, [1, 2, 3], seed=6)
    cfgd, w = plain.read_model_dir(sharp_dirs[name])
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": toks[:1], "want": [0]} for rid, toks in reqs],
              "end": ["r0"]},
             {"step": 1, "entries": [{"id": rid, "tokens": toks[1:2], "want": [0]} for rid, toks in reqs[1:]],
              "end": ["r1"]},
             {"step": 2, "entries": [{"id": "r2", "tokens": reqs[2][1][2:], "want": [0]},
                                     {"id": "w", "tokens": reqs[2][1], "want": [0, 1, 2]}], "end": ["r2", "w"]}]
    runner = _runner(sharp_dirs[name], dtype, 8, 8)
    rp = TraceReplayer(runner)
    got = rc.collect(steps, {s["step"]: rp.run_step(s) for s in steps})
    for rid, toks in reqs + [("w", reqs[2][1])]:
        want = plain.forward_logits(cfgd, w, toks).numpy()
        for p in range(len(toks)):
            assert np.abs(got[(rid, p)] - want[p]).max() <= TOL_SHARP[dtype] * np.abs(want).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d"])
def test_decode_steps_replayed_from_cuda_graphs(model_dirs, name, dtype):
    """With CUDA graphs on, steps made of single tokens are replayed from a graph of their
    row-count bucket (padded with rows that write to a scratch page); the logits still
    equal the plain implementation's, in a trace that mixes such steps with prompt portions
    and that hands pages from finished requests to new ones."""
    from emberserve_b200.engine.replay import TraceReplayer

    cfg = ALL[name]
    reqs = rc.make_requests(cfg.vocab_size, [30, 41, 17, 55, 23, 38], seed=12)
    cfgd, w = plain.read_model_dir(model_dirs[name])
    steps = rc.mixed(reqs, max_live=3, seed=2, decode_tail=20)
    ps = PAGE_SIZES[name]
    runner = _runner(model_dirs[name], dtype, ps, TraceReplayer.pages_for(rc.max_live_tokens(steps), ps))
    assert runner.enable_graphs(cfg.max_position_embeddings, 4)
    rp = TraceReplayer(runner)
    got = rc.collect(steps, {s["step"]: rp.run_step(s) for s in steps})
    assert runner.graphs._graphs, "no step went through a graph"
    assert {1, 2, 4} & set(runner.graphs._graphs), sorted(runner.graphs._graphs)
    for rid, toks in reqs:
        want = plain.forward_logits(cfgd, w, toks).numpy()
        err = max(float(np.abs(got[(rid, p)] - want[p]).max()) for p in range(len(toks)))
        assert err <= TOL[dtype] * float(np.abs(want).max()), (rid, err)
    runner.cache.check()


# ---- the cache sized from free memory ---------------------------------------------------------------

def test_cache_from_free_memory_leaves_room_for_the_graphs_and_the_largest_steps():
    """The 7B shape with 97 % of the free memory in use, 256 sequences and a step budget of 8,192
    tokens: the cache is sized first, the graphs of all row buckets are captured after it, then the
    largest prompt portion and the largest decode step run.  A reserve that forgot the graphs'
    scratch and logits, or the activations of a full portion, runs out of memory here."""
    import gc

    from emberserve_b200.config.engine import EngineConfig
    from emberserve_b200.config.model import Qwen2Config
    from emberserve_b200.engine.llm_engine import LLMEngine
    from emberserve_b200.engine.runner import ModelRunner, StepRow

    gc.collect()
    torch.cuda.empty_cache()
    cfg = Qwen2Config(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                      num_attention_heads=28, num_key_value_heads=4, head_dim=128, max_position_embeddings=32768,
                      rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False, attention_bias=True,
                      eos_token_ids=(151645,))
    ecfg = EngineConfig(dtype=torch.bfloat16, gpu_memory_utilization=0.97, max_num_seqs=256, max_model_len=32768,
                        max_num_batched_tokens=8192)
    runner = ModelRunner.from_random(cfg, seed=0, dtype=torch.bfloat16, device=DEV,
                                     **LLMEngine.runner_options(ecfg))
    plan = runner.memory_plan
    assert plan is not None and runner.num_pages == plan.num_pages > 100_000
    assert plan.step_scratch == 8192 * runner.decoder.scratch_bytes_per_token(2) and plan.graph_logits == 256 * 152064 * 4
    assert runner.storage.bytes() == (runner.num_pages + 1) * plan.bytes_per_page
    free_after_cache = torch.cuda.mem_get_info(DEV)[0]
    assert free_after_cache >= plan.reserve  # what was kept for the steps is still there
    engine = LLMEngine.from_runner(runner, ecfg)  # captures the graphs of all 14 buckets
    assert sorted(runner.graphs._graphs) == [1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256]
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg.vocab_size, (8192 + 256,), generator=g).tolist()
    runner.cache.admit(0, 8192)
    logits = runner.step([StepRow(0, toks[:8192], 0, [8191])])  # the largest prompt portion
    assert torch.isfinite(logits).all()
    for s in range(1, 256):
        runner.cache.admit(s, 1)
    runner.cache.extend(0, 8193)
    rows = [StepRow(0, [toks[8192]], 8192, [0])] + [StepRow(s, [toks[8192 + s]], 0, [0]) for s in range(1, 256)]
    logits = runner.step(rows)  # the largest decode step, from the graph of 256 rows
    assert logits.shape == (256, cfg.vocab_size) and torch.isfinite(logits).all()
    torch.cuda.synchronize()
    # the steps stayed inside what was kept for them (the utilization's own 3 % is never touched)
    used_by_steps = free_after_cache - torch.cuda.mem_get_info(DEV)[0]
    assert used_by_steps <= plan.reserve, (used_by_steps, plan.reserve)
    del engine, runner, logits
    gc.collect()
    torch.cuda.empty_cache()


def test_a_request_wider_than_the_graphs_tables_decodes_eagerly(model_dirs):
    """Graphs are captured for contexts up to a maximum; a request that holds more pages than
    their block tables are wide (pages were reserved for its whole prompt at admission) takes the
    eager path instead of overflowing the graph's static buffer, and its logits are right; a
    request that fits goes through the graph in the same run."""
    from emberserve_b200.engine.runner import StepRow

    name = "tiny_b"
    cfg = ALL[name]
    (_, long_toks), (_, short_toks) = rc.make_requests(cfg.vocab_size, [90, 20], seed=21)
    cfgd, w = plain.read_model_dir(model_dirs[name])
    runner = _runner(model_dirs[name], torch.float32, PAGE_SIZES[name], 32)
    assert runner.enable_graphs(32, 4)  # graphs for contexts of at most 32 tokens: tables of 4 pages of 8
    runner.cache.admit(0, 90)   # 12 pages from the start
    runner.cache.admit(1, 12)
    got = {0: [], 1: []}
    runner.step([StepRow(0, long_toks[:10], 0, []), StepRow(1, short_toks[:12], 0, [])])
    for i in range(6):  # both decode; request 0 stands at position 10..15, well inside the graphs' range
        runner.cache.extend(1, 13 + i)
        rows = [StepRow(0, [long_toks[10 + i]], 10 + i, [0]), StepRow(1, [short_toks[12 + i]], 12 + i, [0])]
        assert not runner.graphs.usable(rows) and runner.graphs.usable(rows[1:])
        out = runner.step(rows).cpu().numpy()
        got[0].append(out[0])
        got[1].append(out[1])
    for seq, toks, first in ((0, long_toks, 10), (1, short_toks, 12)):
        want = plain.forward_logits(cfgd, w, toks[:first + 6]).numpy()
        for i in range(6):
            assert np.abs(got[seq][i] - want[first + i]).max() <= TOL[torch.float32] * np.abs(want).max()
    runner.cache.extend(1, 19)
    runner.step([StepRow(1, [short_toks[18]], 18, [0])])  # alone it replays a graph
    assert 1 in runner.graphs._graphs
    runner.cache.check()


# ---- faults that random weights would hide ------------------------------------------------------

def _with_attention_pointing_at(model_dir, out_dir, gain=5.0):
    """A copy of a model whose q and k projections are scaled up (scores grow with the
    square of the gain) so that attention is peaked instead of nearly uniform: the result at
    a position then hangs on few keys, near or far, and a missed key shows."""
    from safetensors.torch import load_file, save_file

    out_dir.mkdir(parents=True, exist_ok=True)
    (out_dir / "config.json").write_text((model_dir / "config.json").read_text())
    t = load_file(str(model_dir / "model.safetensors"))
    for k in t:
        if ".q_proj." in k or ".k_proj." in k:
            t[k] = (t[k].float() * gain).to(t[k].dtype)
    save_file(t, str(out_dir / "model.safetensors"))
    return out_dir


@pytest.mark.parametrize("name", ["tiny_b", "tiny_c", "tiny_d"])
def test_peaked_attention_far_keys_window_edge_page_edge(model_dirs, tmp_path, name):
    """With peaked attention a skipped key, an off-by-one at the window's edge or a wrong
    slot at a page's edge changes logits by far more than the tolerance.  The sequence is
    cut so that portions start and end on and around page edges and the window's edge."""
    from emberserve_b200.engine.replay import TraceReplayer

    folder = _with_attention_pointing_at(model_dirs[name], tmp_path / "peaked")
    cfg = ALL[name]
    ps = PAGE_SIZES[name]
    n = min(cfg.max_position_embeddings - 1, 230)
    reqs = rc.make_requests(cfg.vocab_size, [n], seed=8)
    cfgd, w = plain.read_model_dir(folder)
    want = plain.forward_logits(cfgd, w, reqs[0][1]).numpy()
    # the attention must really be peaked, else the test shows nothing
    base = plain.forward_logits(*plain.read_model_dir(model_dirs[name]), reqs[0][1]).numpy()
    assert np.abs(want - base).max() > 0.2 * np.abs(want).max()
    win = cfg.sliding_window or 24
    cuts = sorted({ps - 1, ps, ps + 1, 2 * ps, win - 1, win, win + 1, 3 * ps + 1, 64, 65, 96, 127, 128, 129, n})
    toks = reqs[0][1]
    steps, prev = [], 0
    for c in cuts:
        if c <= prev or c > n:
            continue
        steps.append({"entries": [{"id": "r0", "tokens": toks[prev:c], "want": list(range(c - prev))}], "end": []})
        prev = c
    for i, s in enumerate(steps):
        s["step"] = i
    for dtype in (torch.float32, torch.bfloat16):
        runner = _runner(folder, dtype, ps, -(-n // ps) + 1)
        rp = TraceReplayer(runner)
        got = rc.collect(steps, {s["step"]: rp.run_step(s) for s in steps})
        err = max(float(np.abs(got[("r0", p)] - want[p]).max()) for p in range(n))
        assert err <= TOL_SHARP[dtype] * float(np.abs(want).max()), (dtype, err)


def test_stale_page_contents_do_not_leak(sharp_dirs):
    """A pool of exactly the pages one request needs: the second request gets the first
    one's pages, full of its keys, and must not see them."""
    from emberserve_b200.engine.replay import TraceReplayer

    name = "tiny_a"
    reqs = rc.make_requests(ALL[name].vocab_size, [37, 35], seed=9)
    cfgd, w = plain.read_model_dir(sharp_dirs[name])
    steps = rc.portions(reqs)
    runner = _runner(sharp_dirs[name], torch.float32, 4, 10)
    rp = TraceReplayer(runner)
    got = rc.collect(steps, {s["step"]: rp.run_step(s) for s in steps})
    for rid, toks in reqs:
        want = plain.forward_logits(cfgd, w, toks).numpy()
        for p in range(len(toks)):
            assert np.abs(got[(rid, p)] - want[p]).max() <= TOL[torch.float32] * np.abs(want).max()


# ---- each part alone ----------------------------------------------------------------------------

def _ctx(q_lens, starts, dtype):
    from emberserve_b200.engine.runner import ScratchArena
    from emberserve_b200.parts.base import StepContext

    b, n = len(q_lens), sum(q_lens)
    i32 = dict(dtype=torch.int32, device=DEV)
    pos = torch.cat([torch.arange(s, s + q) for s, q in zip(starts, q_lens)]).to(**i32)
    row = torch.repeat_interleave(torch.arange(b), torch.tensor(q_lens)).to(**i32)
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), **i32)
    return StepContext(num_tokens=n, num_rows=b, dtype=dtype, device=torch.device(DEV),
                       tokens=torch.zeros(n, **i32), positions=pos, row_of_token=row, cu_q=cu,
                       starts=torch.tensor(starts, **i32), q_lens=q_lens, start_list=starts,
                       max_q_len=max(q_lens), max_ctx_len=max(s + q for s, q in zip(starts, q_lens)),
                       scratch=ScratchArena(torch.device(DEV)))


def _bind_random(part, dtype, seed, std=0.3):
    g = torch.Generator().manual_seed(seed)
    params, by_source = {}, {}
    for local, ps in part.param_specs().items():
        t = torch.ones(ps.shape) if ps.init == "ones" else torch.randn(ps.shape, generator=g) * std
        if ps.init == "ones":
            t = t + 0.1 * torch.randn(ps.shape, generator=g)
        t = t.to(dtype)
        params[local] = t.to(DEV)
        for src in ps.sources:
            by_source[src.name] = (t if src.rows is None else t[src.rows[0]:src.rows[1]]).double()
    part.bind(params)
    return by_source


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_norm_part_alone(dtype):
    from emberserve_b200.parts.base import build_part
    from emberserve_b200.parts.norm import RMSNormSpec

    part = build_part("norm", RMSNormSpec(200, 3e-5, "n.weight"), "n")
    w = _bind_random(part, dtype, 0)
    ctx = _ctx([5, 1], [0, 9], dtype)
    g = torch.Generator().manual_seed(1)
    delta = torch.randn(6, 200, generator=g).to(dtype)
    res = torch.randn(6, 200, generator=g)
    r = res.to(DEV)
    out = part.forward(delta.to(DEV), r, ctx)
    want_res = res.double() + delta.double()
    want = plain.rms_norm(want_res, w["n.weight"], 3e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(r.double().cpu(), want_res, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(out.double().cpu(), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("rows,hidden,inter", [(8, 256, 384), (1, 3584, 1024), (13, 200, 128)])
@pytest.mark.parametrize("consumer", ["plain", "gated", "float32 weight"])
def test_norm_split_between_the_products_around_it(rows, hidden, inter, consumer):
    """A sub-layer's last product, asked to begin the norm behind it, and the product behind the
    norm that finishes it (a plain one, the gated one, and one whose weight is stored in 32 bits,
    which finishes the norm the plain way) against the chain product -> norm kernel -> product."""
    from emberserve_b200.parts.base import ScaledRows, build_part
    from emberserve_b200.parts.linear import gated_linear, linear
    from emberserve_b200.parts.norm import RMSNormSpec

    dtype = torch.bfloat16
    g = torch.Generator(device=DEV).manual_seed(rows + hidden)
    norm = build_part("norm", RMSNormSpec(hidden, 1e-5, "n.weight"), "n")
    norm.bind({"weight": (1 + 0.2 * torch.randn(hidden, device=DEV, generator=g)).to(dtype)})
    ctx = _ctx([1] * rows, list(range(rows)), dtype)
    x = torch.randn(rows, 512, device=DEV, generator=g).to(dtype)
    w1 = (torch.randn(hidden, 512, device=DEV, generator=g) * 0.05).to(dtype)
    res0 = torch.randn(rows, hidden, device=DEV, generator=g)
    n_out = 2 * inter if consumer == "gated" else inter
    w2 = (torch.randn(n_out, hidden, device=DEV, generator=g) * 0.05).to(torch.float32 if consumer == "float32 weight" else dtype)
    bias = None if consumer == "gated" else torch.randn(n_out, device=DEV, generator=g).to(w2.dtype)

    def behind_the_norm(x_in, out):
        if consumer == "gated":
            assert gated_linear(x_in, w2, out)
        else:
            linear(x_in, w2, bias, out, ctx.scratch)
        return out.float().clone()

    # the chain of three kernels
    res_a = res0.clone()
    delta = linear(x, w1, None, torch.empty(rows, hidden, dtype=dtype, device=DEV), ctx.scratch)
    normed = norm.forward(delta, res_a, ctx).clone()
    want = behind_the_norm(normed, torch.empty(rows, inter, dtype=dtype, device=DEV))
    # the norm split between the two products
    res_b = res0.clone()
    request = norm.split_request(res_b, ctx)
    assert request is not None
    rows_b = linear(x, w1, None, torch.empty(rows, hidden, dtype=dtype, device=DEV), ctx.scratch, request)
    assert isinstance(rows_b, ScaledRows) and norm.forward(rows_b, res_b, ctx) is rows_b
    torch.testing.assert_close(res_b, res_a, rtol=0, atol=2e-2 * float(delta.float().abs().max()))  # (unrounded delta)
    torch.testing.assert_close(rows_b.materialize().float(), normed.float(), rtol=2e-2, atol=2e-2)
    got = behind_the_norm(rows_b, torch.empty(rows, inter, dtype=dtype, device=DEV))
    assert float((got - want).abs().max()) <= 2e-2 * float(want.abs().max()) + 1e-3
    # a step of more rows than the products take a norm for: no request, the norm is a kernel
    assert norm.split_request(torch.zeros(17, hidden, device=DEV), _ctx([17], [0], dtype)) is None
    assert norm.split_request(res_b.float(), _ctx([1] * rows, list(range(rows)), torch.float32)) is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_feed_forward_part_alone(dtype):
    from emberserve_b200.parts.base import build_part
    from emberserve_b200.parts.mlp import SwiGLUSpec

    part = build_part("feed_forward", SwiGLUSpec(72, 200, "m.gate_proj", "m.up_proj", "m.down_proj"), "m")
    w = _bind_random(part, dtype, 2, std=0.1)
    ctx = _ctx([7], [0], dtype)
    x = torch.randn(7, 72, generator=torch.Generator().manual_seed(3)).to(dtype)
    out = part.forward(x.to(DEV), ctx)
    want = plain.swiglu(x.double(), w, "m")
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    torch.testing.assert_close(out.double().cpu(), want, rtol=tol, atol=tol * float(want.abs().max()))


def test_position_part_alone():
    from emberserve_b200.parts.base import build_part
    from emberserve_b200.parts.rope import RotarySpec

    part = build_part("position", RotarySpec(48, 50000.0, 300), "p")
    table, rot = part.rotary(torch.device(DEV))
    assert rot == 48 and table.shape == (300, 24, 2) and part.max_positions == 300
    ang = plain.rope_angles(torch.arange(300), 48, 50000.0)[:, :24].double()
    torch.testing.assert_close(table[..., 0].double().cpu(), ang.cos(), rtol=0, atol=2e-6)
    torch.testing.assert_close(table[..., 1].double().cpu(), ang.sin(), rtol=0, atol=2e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_alone_in_two_steps(dtype, window):
    """The mixer alone: a sequence in two portions through a paged cache with scattered
    pages equals the plain attention block on the whole sequence."""
    from emberserve_b200.parts.attention import AttentionSpec
    from emberserve_b200.parts.base import PagedKVHandle, build_part
    from emberserve_b200.parts.rope import RotarySpec

    hidden, nh, nkv, d, ps, t = 80, 6, 2, 32, 4, 27
    spec = AttentionSpec(hidden, nh, nkv, d, True, RotarySpec(d, 1e4, 64), "a.q_proj", "a.k_proj", "a.v_proj",
                         "a.o_proj", window=window)
    part = build_part("mixer", spec, "a")
    assert part.cache_need().window == window and part.cache_need().num_kv_heads == nkv
    w = _bind_random(part, dtype, 4, std=0.25)
    x = torch.randn(t, hidden, generator=torch.Generator().manual_seed(5)).to(dtype)
    g = dict(heads=nh, kv_heads=nkv, head_dim=d, theta=1e4, bias=True)
    want = plain.attention_block(x.double(), w, "a", g, torch.arange(t), window)
    pages = 16
    kc = torch.full((pages, nkv, ps, d), 50.0, dtype=dtype, device=DEV)
    vc = torch.full((pages, nkv, ps, d), 50.0, dtype=dtype, device=DEV)
    bt = torch.tensor([[11, 3, 8, 0, 14, 6, 9]], dtype=torch.int32, device=DEV)
    outs = []
    for lo, hi in ((0, 10), (10, t)):
        ctx = _ctx([hi - lo], [lo], dtype)
        outs.append(part.forward(x[lo:hi].to(DEV), ctx, PagedKVHandle(kc, vc, bt, ps, window, True)).clone())
    got = torch.cat(outs).double().cpu()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    torch.testing.assert_close(got, want, rtol=tol, atol=tol * float(want.abs().max()))


def test_block_part_alone():
    from emberserve_b200.parts.attention import AttentionSpec
    from emberserve_b200.parts.base import PagedKVHandle, build_part
    from emberserve_b200.parts.block import PreNormBlockSpec
    from emberserve_b200.parts.mlp import SwiGLUSpec
    from emberserve_b200.parts.norm import RMSNormSpec
    from emberserve_b200.parts.rope import RotarySpec

    hidden, t, p = 48, 13, "model.layers.0"
    spec = PreNormBlockSpec(
        mixer=AttentionSpec(hidden, 3, 3, 16, False, RotarySpec(16, 1e4, 32), f"{p}.self_attn.q_proj",
                            f"{p}.self_attn.k_proj", f"{p}.self_attn.v_proj", f"{p}.self_attn.o_proj"),
        feed_forward=SwiGLUSpec(hidden, 100, f"{p}.mlp.gate_proj", f"{p}.mlp.up_proj", f"{p}.mlp.down_proj"),
        mixer_norm=RMSNormSpec(hidden, 1e-5, f"{p}.input_layernorm.weight"),
        ffn_norm=RMSNormSpec(hidden, 1e-5, f"{p}.post_attention_layernorm.weight"))
    block = build_part("block", spec, "layers.0")
    w = {}
    for i, child in enumerate(block.children().values()):
        w.update(_bind_random(child, torch.float32, 10 + i, std=0.2))
    h0 = torch.randn(t, hidden, generator=torch.Generator().manual_seed(6))
    g = dict(heads=3, kv_heads=3, head_dim=16, theta=1e4, bias=False, eps=1e-5, window=None, max_window_layers=0)
    want = plain.decoder_layer(h0.double(), w, 0, g, torch.arange(t))
    kc = torch.zeros(4, 3, 8, 16, device=DEV)
    vc = torch.zeros_like(kc)
    bt = torch.tensor([[2, 1]], dtype=torch.int32, device=DEV)
    ctx = _ctx([t], [0], torch.float32)
    residual = h0.to(DEV).clone()
    delta = block.forward(None, residual, ctx, PagedKVHandle(kc, vc, bt, 8, None, True))
    got = (residual + delta).double().cpu()  # the next norm would perform this add
    torch.testing.assert_close(got, want, rtol=2e-5, atol=2e-5)


# ---- a toy architecture with a mixer that keeps state of its own ----------------------------------

def _toy_decay_architecture(tmp_path):
    """Registers a toy architecture whose layers alternate between a recurrent toy mixer with
    state of its own (s_t = decay * s_{t-1} + x_t W_in ; y_t = s_t W_out) and attention, with a
    toy norm before the toy mixers and the head; writes a random model folder.  Returns
    (config, folder, plain float64 restatement)."""
    from emberserve_b200.config.model import ModelConfig
    from emberserve_b200.engine.replay import TraceReplayer
    from emberserve_b200.engine.runner import ModelRunner
    from emberserve_b200.parts.attention import AttentionSpec
    from emberserve_b200.parts.base import FixedState, Mixer, Norm, ParamSpec, Source, register_part
    from emberserve_b200.parts.block import PreNormBlockSpec
    from emberserve_b200.parts.decoder import DecoderSpec, LayerCall
    from emberserve_b200.parts.mlp import SwiGLUSpec
    from emberserve_b200.parts.norm import RMSNormSpec
    from emberserve_b200.parts.rope import RotarySpec
    from emberserve_b200.registry import register_architecture
    from emberserve_b200.weights.loader import write_random_model

    @dataclass(frozen=True)
    class ToyDecaySpec:
        hidden: int
        state: int
        decay: float
        name: str
        kind: str = "toy_decay"

    @register_part("mixer", "toy_decay")
    class ToyDecay(Mixer):
        def cache_need(self):
            return FixedState((self.spec.state,), "float32")

        def param_specs(self):
            s = self.spec
            return {"w_in": ParamSpec((s.state, s.hidden), [Source(s.name + ".in.weight")]),
                    "w_out": ParamSpec((s.hidden, s.state), [Source(s.name + ".out.weight")])}

        def forward(self, x, ctx, cache):
            u = x.float() @ self.w_in.float().t()
            if ctx.all_decode:
                # a step of single tokens: nothing is read on the host, so that the step can be
                # captured in a CUDA graph (rows that pad a graph share a scratch slot)
                idx = cache.slots.long()
                s = self.spec.decay * cache.state.index_select(0, idx) + u
                cache.state.index_copy_(0, idx, s)
                return (s @ self.w_out.float().t()).to(x.dtype)
            y = torch.empty_like(u)
            slots = cache.slots.tolist()
            n0 = 0
            for row, q in enumerate(ctx.q_lens):  # a request's tokens in order, from its state
                s = cache.state[slots[row]]
                for i in range(n0, n0 + q):
                    s = self.spec.decay * s + u[i]
                    y[i] = s
                cache.state[slots[row]] = s
                n0 += q
            return (y @ self.w_out.float().t()).to(x.dtype)

    @dataclass(frozen=True)
    class ToyLayerNormSpec:
        dim: int
        eps: float
        name: str
        kind: str = "toy_layernorm"

    @register_part("norm", "toy_layernorm")
    class ToyLayerNorm(Norm):
        """Mean-centred norm with gain and bias, written to the documented Norm interface only
        (delta, residual, ctx, rows): it stands before the toy mixers and before the head."""

        def param_specs(self):
            s = self.spec
            return {"gain": ParamSpec((s.dim,), [Source(s.name + ".weight")], init="ones"),
                    "bias": ParamSpec((s.dim,), [Source(s.name + ".bias")], init="bias")}

        def forward(self, delta, residual, ctx, rows=None):
            if rows is None:
                if delta is not None:
                    residual += delta.float()
                r = residual
            else:
                r = residual[rows.long()]
                if delta is not None:
                    r = r + delta[rows.long()].float()
            r = r - r.mean(-1, keepdim=True)
            y = r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + self.spec.eps)
            return (y * self.gain.float() + self.bias.float()).to(ctx.dtype)

    def plain_layer_norm(h, gain, bias, eps):
        r = h - h.mean(-1, keepdim=True)
        return r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + eps) * gain + bias

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyDecayForCausalLM"
        vocab_size: int = 90
        hidden_size: int = 48
        state_size: int = 20
        num_layers: int = 4
        decay: float = 0.8

        @classmethod
        def from_dict(cls, cfg):
            return cls(**{f.name: cfg[f.name] for f in dataclasses.fields(cls) if f.name in cfg})

        def to_dict(self):
            return dict(dataclasses.asdict(self), architectures=[self.architecture])

    def build(cfg: ToyConfig) -> DecoderSpec:
        layers = []
        for i in range(cfg.num_layers):
            p = f"toy.{i}"
            mixer = (ToyDecaySpec(cfg.hidden_size, cfg.state_size, cfg.decay, f"{p}.rec") if i % 2 == 0 else
                     AttentionSpec(cfg.hidden_size, 3, 1, 16, False, RotarySpec(16, 1e4, 128), f"{p}.q", f"{p}.k",
                                   f"{p}.v", f"{p}.o"))
            layers.append(PreNormBlockSpec(
                mixer=mixer, feed_forward=SwiGLUSpec(cfg.hidden_size, 64, f"{p}.g", f"{p}.u", f"{p}.d"),
                mixer_norm=(ToyLayerNormSpec(cfg.hidden_size, 1e-4, f"{p}.n1") if i % 2 == 0 else
                            RMSNormSpec(cfg.hidden_size, 1e-5, f"{p}.n1")),
                ffn_norm=RMSNormSpec(cfg.hidden_size, 1e-5, f"{p}.n2")))
        return DecoderSpec(vocab_size=cfg.vocab_size, hidden=cfg.hidden_size, embed_name="toy.embed",
                           layers=layers, order=[LayerCall(i, i) for i in range(cfg.num_layers)],
                           final_norm=ToyLayerNormSpec(cfg.hidden_size, 1e-4, "toy.norm"), head_name=None,
                           max_positions=128)

    register_architecture("ToyDecayForCausalLM", ToyConfig, build)
    cfg = ToyConfig()
    folder = write_random_model(cfg, tmp_path / "toy", seed=3, std=0.15, store_dtype=torch.float32)

    def plain_toy(tokens):
        from safetensors.torch import load_file

        w = {k: v.double() for k, v in load_file(str(folder / "model.safetensors")).items()}
        h = w["toy.embed"][torch.tensor(tokens)]
        t = len(tokens)
        for i in range(cfg.num_layers):
            p = f"toy.{i}"
            if i % 2 == 0:
                x = plain_layer_norm(h, w[f"{p}.n1.weight"], w[f"{p}.n1.bias"], 1e-4)
                u = x @ w[f"{p}.rec.in.weight"].T
                s = torch.zeros(cfg.state_size, dtype=torch.float64)
                ys = []
                for j in range(t):
                    s = cfg.decay * s + u[j]
                    ys.append(s)
                a = torch.stack(ys) @ w[f"{p}.rec.out.weight"].T
            else:
                x = plain.rms_norm(h, w[f"{p}.n1"], 1e-5)
                q = (x @ w[f"{p}.q.weight"].T).view(t, 3, 16)
                k = (x @ w[f"{p}.k.weight"].T).view(t, 1, 16)
                v = (x @ w[f"{p}.v.weight"].T).view(t, 1, 16)
                ang = plain.rope_angles(torch.arange(t), 16, 1e4)
                a = plain.causal_attention(plain.apply_rope(q, ang), plain.apply_rope(k, ang), v)
                a = a.reshape(t, 48) @ w[f"{p}.o.weight"].T
            h = h + a
            y = plain.rms_norm(h, w[f"{p}.n2"], 1e-5)
            gate, up = y @ w[f"{p}.g.weight"].T, y @ w[f"{p}.u.weight"].T
            h = h + (torch.nn.functional.silu(gate) * up) @ w[f"{p}.d.weight"].T
        return (plain_layer_norm(h, w["toy.norm.weight"], w["toy.norm.bias"], 1e-4) @ w["toy.embed"].T).numpy()
    return cfg, folder, plain_toy


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """A recurrent toy mixer and a toy norm defined HERE are registered as parts, used by a toy
    architecture registered HERE, written as a random model folder, loaded, and stepped in
    portions, token by token and beside another request.  Nothing in the package is edited
    for it."""
    from emberserve_b200.engine.replay import TraceReplayer
    from emberserve_b200.engine.runner import ModelRunner

    cfg, folder, plain_toy = _toy_decay_architecture(tmp_path)
    runner = ModelRunner.from_dir(folder, torch.float32, device=DEV, page_size=8, num_pages=24,
                                  num_state_slots=2)
    kinds = [type(g.need).__name__ for g in runner.groups]
    assert sorted(kinds) == ["FixedState", "PagedKV"]
    reqs = rc.make_requests(cfg.vocab_size, [21, 30, 17], seed=2)
    want = {rid: plain_toy(toks) for rid, toks in reqs}
    for steps in (rc.whole(reqs), rc.portions(reqs), rc.mixed(reqs, max_live=2, seed=1, decode_tail=5)):
        rp = TraceReplayer(runner)
        got = rc.collect(steps, {s["step"]: rp.run_step(s) for s in steps})
        for rid, toks in reqs:
            for p in range(len(toks)):
                assert np.abs(got[(rid, p)] - want[rid][p]).max() <= 3e-5 * np.abs(want[rid]).max()
        runner.cache.check()
        assert runner.cache.stats().free_state_slots == 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_toy_mixer_with_state_decodes_from_cuda_graphs(tmp_path, dtype):
    """The same toy architecture with CUDA graphs on: the state slot of each row and the slots
    to be zeroed reach the captured step through its static integers, padded rows use a scratch
    slot, and a slot that goes from a finished request to a new one starts from zero."""
    from emberserve_b200.engine.replay import TraceReplayer
    from emberserve_b200.engine.runner import ModelRunner

    cfg, folder, plain_toy = _toy_decay_architecture(tmp_path)
    reqs = rc.make_requests(cfg.vocab_size, [21, 30, 17, 26, 1, 19], seed=5)
    steps = rc.mixed(reqs, max_live=3, seed=4, decode_tail=12)
    runner = ModelRunner.from_dir(folder, dtype, device=DEV, page_size=8,
                                  num_pages=TraceReplayer.pages_for(rc.max_live_tokens(steps), 8), num_state_slots=3)
    assert runner.enable_graphs(128, 4)
    rp = TraceReplayer(runner)
    got = rc.collect(steps, {s["step"]: rp.run_step(s) for s in steps})
    assert {1, 2, 4} & set(runner.graphs._graphs), "no step went through a graph"
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for rid, toks in reqs:
        want = plain_toy(toks)
        err = max(float(np.abs(got[(rid, p)] - want[p]).max()) for p in range(len(toks)))
        assert err <= tol * float(np.abs(want).max()), (rid, err)
    runner.cache.check()
    assert runner.cache.stats().free_state_slots == 3


# ---- a toy architecture with routed experts, learned positions and a shared cache entry -----------

def test_toy_routing_learned_positions_and_shared_cache_entry(tmp_path):
    """Three more kinds of part defined HERE, none of them a model of anyone's: a feed-forward
    that routes every token to 2 of 4 small experts (router logits and their softmax in 32
    bits), a position encoding that adds a learned vector per position to the embedding
    (attention then runs without rotary), and an order of layers that names layer 0 twice
    (its weights at two depths, a cache entry for each) and lets the last call read the keys
    and values that layer 1 wrote instead of writing its own.  Built from a random model
    folder and replayed under every cut against a plain float64 restatement."""
    from emberserve_b200.config.model import ModelConfig
    from emberserve_b200.engine.replay import TraceReplayer
    from emberserve_b200.engine.runner import ModelRunner
    from emberserve_b200.parts.attention import AttentionSpec
    from emberserve_b200.parts.base import FeedForward, ParamSpec, PositionEncoding, Source, register_part
    from emberserve_b200.parts.block import PreNormBlockSpec
    from emberserve_b200.parts.decoder import DecoderSpec, LayerCall
    from emberserve_b200.parts.mlp import SwiGLUSpec
    from emberserve_b200.parts.norm import RMSNormSpec
    from emberserve_b200.registry import register_architecture
    from emberserve_b200.weights.loader import write_random_model

    @dataclass(frozen=True)
    class ToyExpertsSpec:
        hidden: int
        inter: int
        experts: int
        top_k: int
        name: str
        kind: str = "toy_top_k_experts"

    @register_part("feed_forward", "toy_top_k_experts")
    class ToyExperts(FeedForward):
        def param_specs(self):
            s = self.spec
            specs = {"router": ParamSpec((s.experts, s.hidden), [Source(f"{s.name}.router.weight")])}
            for e in range(s.experts):
                specs[f"up{e}"] = ParamSpec((s.inter, s.hidden), [Source(f"{s.name}.{e}.up.weight")])
                specs[f"down{e}"] = ParamSpec((s.hidden, s.inter), [Source(f"{s.name}.{e}.down.weight")])
            return specs

        def forward(self, x, ctx):
            s = self.spec
            logits = x.float() @ self.router.float().t()  # 32-bit, whatever the activations are
            top, idx = logits.topk(s.top_k, dim=-1)
            gate = torch.softmax(top, dim=-1)
            y = torch.zeros(x.shape[0], s.hidden, dtype=torch.float32, device=x.device)
            for e in range(s.experts):
                weight = (gate * (idx == e)).sum(-1, keepdim=True)  # 0 where the token skips the expert
                h = torch.nn.functional.gelu(x.float() @ getattr(self, f"up{e}").float().t())
                y += weight * (h @ getattr(self, f"down{e}").float().t())
            return y.to(x.dtype)

    @dataclass(frozen=True)
    class ToyLearnedPositionSpec:
        hidden: int
        max_positions: int
        name: str
        kind: str = "toy_learned_position"

    @register_part("position", "toy_learned_position")
    class ToyLearnedPosition(PositionEncoding):
        def param_specs(self):
            s = self.spec
            return {"table": ParamSpec((s.max_positions, s.hidden), [Source(f"{s.name}.weight")])}

        def on_embedding(self, hidden, ctx):
            hidden += self.table.float()[ctx.positions.long()]

        @property
        def max_positions(self):
            return self.spec.max_positions

    @dataclass(frozen=True)
    class ToyRoutedConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyRoutedForCausalLM"
        vocab_size: int = 70
        hidden_size: int = 40
        expert_size: int = 24
        num_experts: int = 4
        experts_per_token: int = 2
        max_positions: int = 96

        @classmethod
        def from_dict(cls, cfg):
            return cls(**{f.name: cfg[f.name] for f in dataclasses.fields(cls) if f.name in cfg})

        def to_dict(self):
            return dict(dataclasses.asdict(self), architectures=[self.architecture])

    heads, kv_heads, head_dim = 2, 1, 16

    def build(cfg: ToyRoutedConfig) -> DecoderSpec:
        def attention(p):
            return AttentionSpec(cfg.hidden_size, heads, kv_heads, head_dim, False, None, f"{p}.q", f"{p}.k",
                                 f"{p}.v", f"{p}.o")

        def routed(p):
            return ToyExpertsSpec(cfg.hidden_size, cfg.expert_size, cfg.num_experts, cfg.experts_per_token, f"{p}.moe")

        layers = []
        for i, ff in enumerate((routed, lambda p: SwiGLUSpec(cfg.hidden_size, 56, f"{p}.g", f"{p}.u", f"{p}.d"),
                                routed)):
            p = f"toy.{i}"
            layers.append(PreNormBlockSpec(mixer=attention(p), feed_forward=ff(p),
                                           mixer_norm=RMSNormSpec(cfg.hidden_size, 1e-5, f"{p}.n1"),
                                           ffn_norm=RMSNormSpec(cfg.hidden_size, 1e-5, f"{p}.n2")))
        order = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(2, 1, write=False)]
        return DecoderSpec(vocab_size=cfg.vocab_size, hidden=cfg.hidden_size, embed_name="toy.embed",
                           layers=layers, order=order, final_norm=RMSNormSpec(cfg.hidden_size, 1e-5, "toy.norm"),
                           head_name="toy.head", max_positions=cfg.max_positions,
                           embedding_position=ToyLearnedPositionSpec(cfg.hidden_size, cfg.max_positions, "toy.pos"))

    register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig, build)
    cfg = ToyRoutedConfig()
    folder = write_random_model(cfg, tmp_path / "toy_routed", seed=8, std=0.2, store_dtype=torch.float32)

    def plain_toy(tokens):
        from safetensors.torch import load_file

        w = {k: v.double() for k, v in load_file(str(folder / "model.safetensors")).items()}
        t = len(tokens)
        h = w["toy.embed"][torch.tensor(tokens)] + w["toy.pos.weight"][:t]
        kept = {}  # cache entry -> (k, v)
        for layer, entry, write in ((0, 0, True), (1, 1, True), (0, 2, True), (2, 1, False)):
            p = f"toy.{layer}"
            x = plain.rms_norm(h, w[f"{p}.n1"], 1e-5)
            q = (x @ w[f"{p}.q.weight"].T).view(t, heads, head_dim)
            if write:
                kept[entry] = ((x @ w[f"{p}.k.weight"].T).view(t, kv_heads, head_dim),
                               (x @ w[f"{p}.v.weight"].T).view(t, kv_heads, head_dim))
            k, v = kept[entry]
            h = h + plain.causal_attention(q, k, v).reshape(t, heads * head_dim) @ w[f"{p}.o.weight"].T
            y = plain.rms_norm(h, w[f"{p}.n2"], 1e-5)
            if layer == 1:
                h = h + (torch.nn.functional.silu(y @ w[f"{p}.g.weight"].T) * (y @ w[f"{p}.u.weight"].T)) @ w[f"{p}.d.weight"].T
                continue
            top, idx = (y @ w[f"{p}.moe.router.weight"].T).topk(cfg.experts_per_token, dim=-1)
            gate = torch.softmax(top, dim=-1)
            out = torch.zeros_like(h)
            for j in range(t):
                for slot in range(cfg.experts_per_token):
                    e = int(idx[j, slot])
                    hid = torch.nn.functional.gelu(y[j] @ w[f"{p}.moe.{e}.up.weight"].T)
                    out[j] += gate[j, slot] * (hid @ w[f"{p}.moe.{e}.down.weight"].T)
            h = h + out
        return (plain.rms_norm(h, w["toy.norm"], 1e-5) @ w["toy.head"].T).numpy()

    runner = ModelRunner.from_dir(folder, torch.float32, device=DEV, page_size=8, num_pages=40)
    assert len(runner.decoder.cache_entries()) == 3 and len(runner.decoder.blocks) == 3
    assert runner.max_positions == cfg.max_positions
    reqs = rc.make_requests(cfg.vocab_size, [23, 31, 18], seed=4)
    want = {rid: plain_toy(toks) for rid, toks in reqs}
    for steps in (rc.whole(reqs), rc.portions(reqs), rc.mixed(reqs, max_live=2, seed=3, decode_tail=6)):
        rp = TraceReplayer(runner)
        got = rc.collect(steps, {s["step"]: rp.run_step(s) for s in steps})
        for rid, toks in reqs:
            for p in range(len(toks)):
                assert np.abs(got[(rid, p)] - want[rid][p]).max() <= 3e-5 * np.abs(want[rid]).max()
        runner.cache.check()
