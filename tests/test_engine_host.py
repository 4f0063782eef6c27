"""Generation through the engine and the Python entry point, on the CPU with the kernels'
restatements: what the scheduler cuts and batches must not change a request's tokens."""

from __future__ import annotations

import pytest
import torch

import kernel_refs
import plain_qwen2 as plain
from host_harness import host_runner
from tiny_configs import ALL, PAGE_SIZES

from emberserve_b200.config.engine import EngineConfig
from emberserve_b200.engine.llm_engine import LLMEngine
from emberserve_b200.engine.request import FinishReason
from emberserve_b200.llm import LLM
from emberserve_b200.sampling.params import SamplingParams


@pytest.fixture(autouse=True)
def _refs(monkeypatch):
    kernel_refs.install(monkeypatch)


def make_llm(model_dir, name, pages=256, **cfg):
    runner = host_runner(model_dir, page_size=PAGE_SIZES[name], num_pages=pages)
    config = EngineConfig(device="cpu", dtype=torch.float32, block_size=PAGE_SIZES[name],
                          max_model_len=ALL[name].max_position_embeddings, **cfg)
    return LLM.from_engine(LLMEngine(runner, config))


def prompts_for(name, lengths, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, ALL[name].vocab_size, (n,), generator=g).tolist() for n in lengths]


def test_greedy_equals_plain_recomputation(model_dirs):
    name = "tiny_a"
    cfg, w = plain.read_model_dir(model_dirs[name])
    prompts = prompts_for(name, [5, 11, 17])
    llm = make_llm(model_dirs[name], name)
    res = llm.generate(prompts, SamplingParams.greedy(8, ignore_eos=True))
    for p, r in zip(prompts, res):
        assert r.output_token_ids == plain.greedy_generate(cfg, w, p, 8)
        assert r.finish_reason == FinishReason.LENGTH and r.prompt_token_ids == p
        assert r.metrics["num_output_tokens"] == 8
    assert [r.request_id for r in res] == ["req-0", "req-1", "req-2"]


@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_batch_equals_alone_and_chunked_equals_unchunked(model_dirs, temperature):
    name = "tiny_b"
    prompts = prompts_for(name, [1, 9, 23, 40], seed=1)
    params = [SamplingParams(max_tokens=12, temperature=temperature, seed=100 + i, ignore_eos=True)
              for i in range(4)]
    base = [r.output_token_ids for r in
            make_llm(model_dirs[name], name, enable_chunked_prefill=False).generate(prompts, params)]
    alone = [make_llm(model_dirs[name], name).generate([p], [sp])[0].output_token_ids
             for p, sp in zip(prompts, params)]
    assert alone == base
    llm = make_llm(model_dirs[name], name, max_num_batched_tokens=7)
    llm.engine.keep_stats = True
    chunked = [r.output_token_ids for r in llm.generate(prompts, params)]
    assert chunked == base
    stats = llm.engine.stats
    assert all(s.num_tokens <= 7 for s in stats)
    assert any(s.num_decode_tokens and s.num_prefill_tokens for s in stats), "no mixed step happened"
    if temperature:
        assert len({tuple(t) for t in base}) == 4  # sampled sequences differ between requests


def test_preemption_preserves_outputs(model_dirs):
    name = "tiny_b"
    prompts = prompts_for(name, [9, 23, 17, 30], seed=2)
    params = [SamplingParams(max_tokens=20, temperature=0.7, seed=i, ignore_eos=True) for i in range(4)]
    roomy = [r.output_token_ids for r in make_llm(model_dirs[name], name).generate(prompts, params)]
    llm = make_llm(model_dirs[name], name, pages=12, max_num_batched_tokens=16)
    llm.engine.keep_stats = True
    tight = [r.output_token_ids for r in llm.generate(prompts, params)]
    assert sum(s.num_preempted for s in llm.engine.stats) >= 1, "the pool was not tight enough"
    assert tight == roomy
    st = llm.engine.runner.cache.stats()
    assert st.num_free == st.num_pages and st.num_sequences == 0


def test_stop_ids_eos_length_and_abort(model_dirs):
    name = "tiny_a"
    cfg, w = plain.read_model_dir(model_dirs[name])
    prompt = prompts_for(name, [6], seed=3)[0]
    free_run = plain.greedy_generate(cfg, w, prompt, 6)
    llm = make_llm(model_dirs[name], name)
    r = llm.generate([prompt], SamplingParams.greedy(6, stop_token_ids=[free_run[2]], ignore_eos=True))[0]
    first = free_run.index(free_run[2])
    assert r.output_token_ids == free_run[:first + 1] and r.finish_reason == FinishReason.STOP
    eng = llm.engine
    eng.eos_token_ids = frozenset({free_run[1]})
    r = llm.generate([prompt], SamplingParams.greedy(6))[0]
    assert r.output_token_ids == free_run[:free_run.index(free_run[1]) + 1]
    assert r.finish_reason == FinishReason.STOP
    eng.add_request("x", prompt, SamplingParams.greedy(50))
    eng.step()
    eng.abort_request("x")
    assert not eng.has_unfinished_requests() and eng.runner.cache.stats().num_sequences == 0
    with pytest.raises(ValueError, match="vocabulary"):
        eng.add_request("y", [ALL[name].vocab_size])
    with pytest.raises(ValueError, match="tokenizer"):
        eng.add_request("z", "text")


def test_max_model_len_ends_a_request(model_dirs):
    name = "tiny_a"
    llm = make_llm(model_dirs[name], name)
    llm.engine.config.max_model_len = 12
    r = llm.generate([prompts_for(name, [8])[0]], SamplingParams.greedy(50, ignore_eos=True))[0]
    assert len(r.output_token_ids) == 4 and r.finish_reason == FinishReason.LENGTH


def test_step_logits_all_positions(model_dirs):
    """The engine's own schedule + step_logits(all_positions) path (the reference's
    check_golden way of reading logits) against the plain implementation."""
    name = "tiny_c"
    cfg, w = plain.read_model_dir(model_dirs[name])
    prompt = prompts_for(name, [50], seed=4)[0]
    eng = make_llm(model_dirs[name], name).engine
    eng.add_request("g", prompt, SamplingParams.greedy(1))
    so = eng.scheduler.schedule()
    logits = eng.step_logits(so, all_positions=True)
    want = plain.forward_logits(cfg, w, prompt, torch.float64)
    assert logits.shape == want.shape
    assert float((logits.double() - want).abs().max()) < 2e-5 * float(want.abs().max())
