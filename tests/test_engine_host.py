"""Generation through the engine and the Python entry point, on the CPU with the kernels'
restatements: what the scheduler cuts and batches must not change a request's tokens."""

from __future__ import annotations

import dataclasses

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


def _mixed_workload(name, model_dir):
    """Requests that end by an end-of-sequence token at different times, by a stop token, by
    max_tokens and by the model length, with sampling and greedy rows."""
    cfg, w = plain.read_model_dir(model_dir)
    prompts = prompts_for(name, [7, 19, 3, 26, 11, 15], seed=9)
    runs = [plain.greedy_generate(cfg, w, p, 10) for p in prompts[:2]]
    params = [
        SamplingParams.greedy(10, stop_token_ids=[runs[0][3]], ignore_eos=True),
        SamplingParams.greedy(10),  # ends at the end-of-sequence token set below
        SamplingParams(max_tokens=9, temperature=0.9, seed=5, ignore_eos=True),
        SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True),
        SamplingParams(max_tokens=14, temperature=0.6, top_k=7, seed=6, ignore_eos=True),
        SamplingParams(max_tokens=60, temperature=0.0, ignore_eos=True),  # the model length ends it
    ]
    return prompts, params, frozenset({runs[1][5]})


@pytest.mark.parametrize("how", [dict(), dict(max_num_batched_tokens=8), dict(pages=7, max_num_batched_tokens=64),
                                 dict(enable_chunked_prefill=False)])
def test_async_scheduling_changes_no_token(model_dirs, how):
    """Launching a step before the tokens of the step before it are read must give the same
    tokens, finish reasons and an empty cache afterwards, whatever ends the requests."""
    name = "tiny_b"
    prompts, params, eos = _mixed_workload(name, model_dirs[name])
    results = []
    for async_on in (False, True):
        llm = make_llm(model_dirs[name], name, async_scheduling=async_on, **how)
        llm.engine.config.max_model_len = 40
        llm.engine.eos_token_ids = eos
        llm.engine.keep_stats = True
        res = llm.generate(prompts, params)
        results.append([(r.output_token_ids, r.finish_reason) for r in res])
        st = llm.engine.runner.cache.stats()
        assert st.num_free == st.num_pages and st.num_sequences == 0
        assert all(t >= 0 for r in res for t in r.output_token_ids)
        if "pages" in how:
            assert sum(s.num_preempted for s in llm.engine.stats) >= 1, "the pool was not tight enough"
    assert results[0] == results[1]
    reasons = [r for _, r in results[0]]
    assert reasons[:2] == [FinishReason.STOP, FinishReason.STOP] and FinishReason.LENGTH in reasons


def test_async_step_returns_the_step_before(model_dirs):
    name = "tiny_a"
    llm = make_llm(model_dirs[name], name)
    eng = llm.engine
    eng.add_request("a", prompts_for(name, [5])[0], SamplingParams.greedy(3, ignore_eos=True))
    outs = [eng.step() for _ in range(4)]
    assert [len(o) for o in outs] == [0, 1, 1, 1]  # the prompt's token arrives with the second call
    assert outs[3][0].finished and not eng.has_unfinished_requests()
    assert eng.step() == []
    # an abort while a token is on its way drops the token
    eng.add_request("b", prompts_for(name, [5])[0], SamplingParams.greedy(5, ignore_eos=True))
    eng.step()
    eng.abort_request("b")
    assert eng.step() == [] and eng.runner.cache.stats().num_sequences == 0


@pytest.mark.parametrize("async_on", [False, True])
def test_request_that_outgrows_the_pool_is_dropped(model_dirs, async_on):
    """Three pages of eight tokens: a prompt of 15 fits, its 30 tokens of output do not.  The
    request preempts itself, can never be admitted again, and ends with ABORT and the tokens it
    had; a request beside it that fits is served."""
    name = "tiny_b"
    prompts = prompts_for(name, [15, 4], seed=6)
    llm = make_llm(model_dirs[name], name, pages=3, async_scheduling=async_on)
    res = llm.generate(prompts, [SamplingParams.greedy(30, ignore_eos=True), SamplingParams.greedy(3, ignore_eos=True)])
    assert res[0].finish_reason == FinishReason.ABORT and 0 < len(res[0].output_token_ids) < 30
    assert res[1].finish_reason == FinishReason.LENGTH and len(res[1].output_token_ids) == 3
    st = llm.engine.runner.cache.stats()
    assert st.num_free == st.num_pages and st.num_sequences == 0


@pytest.mark.parametrize("async_on", [False, True])
def test_a_step_whose_kernel_gave_up_hands_out_no_token(model_dirs, async_on, monkeypatch):
    """A bounded wait of a tcgen05 kernel that runs out leaves a code in the status word.  The
    engine reads the word once it has waited for the step: no token of that step is returned,
    its requests end with ABORT, their pages go back, the word is cleared and the next
    requests are served as if nothing had happened.  (The code is set on the host here; no
    kernel is made to time out.)"""
    import emberserve_b200.kernels as K

    name = "tiny_a"
    word = {"code": 0, "cleared": 0}

    def check_status(clear=True):
        if word["code"]:
            code, word["code"] = word["code"], 0
            word["cleared"] += 1
            raise K.KernelError(f"a wait inside a tcgen05 kernel ran out (code {code})")

    monkeypatch.setattr(K, "check_status", check_status)
    llm = make_llm(model_dirs[name], name, async_scheduling=async_on)
    eng = llm.engine
    prompts = prompts_for(name, [5, 11], seed=3)
    for i, p in enumerate(prompts):
        eng.add_request(f"r{i}", p, SamplingParams.greedy(6, ignore_eos=True))
    seen = []
    for _ in range(2 + async_on):
        seen += eng.step()
    tokens_before = {o.request_id: list(o.output_token_ids) for o in seen}
    word["code"] = 2
    with pytest.raises(K.KernelError, match="ran out"):
        eng.step()
    assert word["cleared"] == 1
    assert not eng.has_unfinished_requests()
    assert eng.step() == []
    for req_id, toks in tokens_before.items():
        assert all(t >= 0 for t in toks)
    eng.runner.cache.check()
    assert eng.runner.cache.num_free_pages(0) == eng.runner.num_pages
    # the engine goes on: the same prompts again give the tokens of an undisturbed run
    again = llm.generate(prompts, SamplingParams.greedy(6, ignore_eos=True))
    clean = make_llm(model_dirs[name], name, async_scheduling=async_on).generate(
        prompts, SamplingParams.greedy(6, ignore_eos=True))
    assert [r.output_token_ids for r in again] == [r.output_token_ids for r in clean]
    assert all(r.finish_reason == FinishReason.LENGTH for r in again)


def test_engine_seed_moves_the_seeds_of_unseeded_requests(model_dirs):
    name = "tiny_b"
    prompts = prompts_for(name, [9, 23], seed=5)
    params = SamplingParams(max_tokens=10, temperature=1.0, ignore_eos=True)  # no seed of its own

    def run(seed):
        return [r.output_token_ids for r in make_llm(model_dirs[name], name, seed=seed).generate(prompts, params)]

    assert run(0) == run(0) and run(7) == run(7)
    assert run(0) != run(7)


def test_from_pretrained_leaves_the_callers_configuration_alone(model_dirs, monkeypatch):
    from emberserve_b200.engine.runner import ModelRunner

    monkeypatch.setattr(ModelRunner, "_require_cuda", False)
    name = "tiny_a"
    cfg = EngineConfig(device="cpu", dtype=torch.float32, block_size=PAGE_SIZES[name], num_gpu_blocks=32,
                       max_model_len=64, enable_cuda_graphs=False)
    before = dataclasses.asdict(cfg)
    eng = LLMEngine.from_pretrained(model_dirs[name], cfg, max_num_seqs=3, dtype="float32")
    assert dataclasses.asdict(cfg) == before
    assert eng.config.max_num_seqs == 3 and eng.config.model_dir == str(model_dirs[name])
    with pytest.raises(TypeError, match="no field"):
        LLMEngine.from_pretrained(model_dirs[name], cfg, no_such_knob=1)


def test_engine_launches_on_its_runners_device_and_checks_the_feedback_size(model_dirs):
    """What the engine launches itself (graph capture, the sampler, events) runs under a device
    guard for the runner's GPU, whichever device is current; on the CPU harness there is nothing
    to guard.  More sequences than sampled tokens can wait on the device are refused."""
    import contextlib
    import types

    from emberserve_b200.engine import runner as runner_module

    name = "tiny_a"
    eng = make_llm(model_dirs[name], name).engine
    assert isinstance(eng._on_device(), contextlib.nullcontext)
    fake = types.SimpleNamespace(runner=types.SimpleNamespace(device=torch.device("cuda", 1)))
    guard = LLMEngine._on_device(fake)
    assert isinstance(guard, torch.cuda.device) and guard.idx == 1
    with pytest.raises(ValueError, match="max_num_seqs"):
        make_llm(model_dirs[name], name, max_num_seqs=runner_module.MAX_DEFERRED_TOKENS + 1)


def test_repetition_penalty_steps_without_lag(model_dirs):
    """A request whose sampling reads its token history keeps the engine on plain stepping,
    and the tokens equal those of an engine with async scheduling off."""
    name = "tiny_a"
    prompts = prompts_for(name, [6, 9], seed=4)
    params = [SamplingParams(max_tokens=8, temperature=0.0, repetition_penalty=1.3, ignore_eos=True),
              SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)]
    a = make_llm(model_dirs[name], name, async_scheduling=True)
    a.engine.add_request("p", prompts[0], params[0])
    assert len(a.engine.step()) == 1  # no lag: the first call already returns the token
    a.engine.reset()
    outs = [[r.output_token_ids for r in make_llm(model_dirs[name], name, async_scheduling=flag).generate(prompts, params)]
            for flag in (True, False)]
    assert outs[0] == outs[1]


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


@pytest.mark.parametrize("seed", range(24))
def test_async_scheduling_under_random_workloads(model_dirs, seed):
    """Random requests (prompt lengths, token limits, stop tokens, sampled and greedy), random
    pool sizes and token budgets, requests added while others run and some aborted on the way:
    async and plain stepping must give every request the same tokens and finish reason, and leave
    the cache empty."""
    import random

    name = "tiny_a"
    rng = random.Random(seed)
    vocab = ALL[name].vocab_size
    n_req = rng.randint(2, 7)
    prompts = [[rng.randrange(vocab) for _ in range(rng.randint(1, 30))] for _ in range(n_req)]
    params = []
    for i in range(n_req):
        stop = [rng.randrange(vocab) for _ in range(rng.randint(0, 6))]
        params.append(SamplingParams(max_tokens=rng.randint(1, 20), temperature=rng.choice([0.0, 0.0, 0.7, 1.2]),
                                     top_k=rng.choice([-1, 5]), top_p=rng.choice([1.0, 0.9]), seed=100 + i,
                                     stop_token_ids=stop, ignore_eos=rng.random() < 0.5))
    eos = frozenset(rng.randrange(vocab) for _ in range(8))
    chunked = rng.random() < 0.7
    how = dict(pages=rng.choice([24, 40, 256]), max_num_batched_tokens=rng.choice([4, 9, 64]) if chunked else 64,
               enable_chunked_prefill=chunked, max_num_seqs=rng.choice([2, 3, 256]))
    arrivals = sorted(rng.randint(0, 12) for _ in range(n_req))  # the step at which each request arrives
    abort_at = {rng.randrange(n_req): rng.randint(1, 15)} if rng.random() < 0.5 else {}

    def run(async_on):
        llm = make_llm(model_dirs[name], name, async_scheduling=async_on, **how)
        eng = llm.engine
        eng.eos_token_ids = eos
        done, step, added = {}, 0, 0
        while added < n_req or eng.has_unfinished_requests():
            while added < n_req and arrivals[added] <= step:
                eng.add_request(f"r{added}", prompts[added], params[added])
                added += 1
            for i, when in abort_at.items():
                if when == step and i < added:
                    eng.abort_request(f"r{i}")
            for out in eng.step():
                if out.finished:
                    done[out.request_id] = (out.output_token_ids, out.finish_reason)
            step += 1
            assert step < 2000, "the engine does not come to an end"
        st = eng.runner.cache.stats()
        assert st.num_free == st.num_pages and st.num_sequences == 0
        eng.runner.cache.check()
        return done

    plain_run, async_run = run(False), run(True)
    aborted = {f"r{i}" for i in abort_at}
    for rid in plain_run.keys() | async_run.keys():
        if rid in aborted:
            continue  # an abort lands a step apart in the two modes; it may or may not come too late
        assert plain_run.get(rid) == async_run.get(rid), rid
    assert all(t >= 0 for toks, _ in async_run.values() for t in toks)


class _LetterTokenizer:
    """Token i is the letter chr(97 + i % 26); tokens 200.. are the two halves of a two-byte
    character, which decodes to U+FFFD until both halves are there."""

    def encode(self, text):
        return [ord(c) - 97 for c in text]

    def decode(self, ids):
        out, i = [], 0
        while i < len(ids):
            if ids[i] == 200:
                if i + 1 < len(ids) and ids[i + 1] == 201:
                    out.append("é")
                    i += 2
                    continue
                out.append("�")
            elif ids[i] != 201:
                out.append(chr(97 + ids[i] % 26))
            i += 1
        return "".join(out)


def test_detokenizer_pieces_stop_strings_and_incomplete_characters():
    from emberserve_b200.engine.detokenizer import Detokenizer, held_back

    assert held_back("xxab", ["abc", "bd"]) == 2 and held_back("xxa", ["b"]) == 0 and held_back("xa", ["ab"]) == 1
    d = Detokenizer(_LetterTokenizer())
    ids, pieces = [], []
    for tok in [0, 1, 2, 23, 24, 3, 4]:  # a b c x y d e ; stop at "xyd"
        ids.append(tok)
        piece, hit = d.feed("r", list(ids), ["xyd", "zz"])
        pieces.append(piece)
        if hit:
            break
    assert hit == "xyd" and "".join(pieces) == "abc"       # the stop string is no part of the text
    assert pieces[3] == "" and pieces[4] == ""             # "x", "xy" were kept back
    d.drop("r")
    # no match in the end: what was kept back comes out with the last piece
    ids, text = [], ""
    for n, tok in enumerate([0, 23, 24, 0]):               # a x y a
        ids.append(tok)
        piece, hit = d.feed("r", list(ids), ["xyd"], final=n == 3)
        text += piece
        assert hit is None
    assert text == "axya"
    # a character whose second half comes a step later is not handed out in halves
    d.drop("r")
    p1, _ = d.feed("r", [0, 200], [])
    p2, _ = d.feed("r", [0, 200, 201], [])
    p3, _ = d.feed("r", [0, 200, 201, 1], [])
    assert (p1, p2, p3) == ("a", "é", "b") or (p1 + p2 + p3 == "aéb" and "�" not in p1 + p2 + p3)
    assert Detokenizer(None).feed("r", [1, 2], ["x"]) == ("", None)


@pytest.mark.parametrize("async_on", [False, True])
def test_stop_strings_end_a_request(model_dirs, async_on):
    """With a tokenizer, a request ends when its text reaches one of its stop strings: the text
    returned ends before the string, the tokens up to the one that completed it are kept, and
    the reason is STOP; a request beside it without stop strings runs on."""
    name = "tiny_a"
    cfg, w = plain.read_model_dir(model_dirs[name])
    prompts = prompts_for(name, [6, 9], seed=8)
    free = plain.greedy_generate(cfg, w, prompts[0], 12)
    tok = _LetterTokenizer()
    text = tok.decode(free)
    stop = text[4:6]                                       # the fifth and sixth characters
    first = text.find(stop)
    llm = make_llm(model_dirs[name], name, async_scheduling=async_on)
    llm.engine.tokenizer = tok
    llm.engine.detokenizer.tokenizer = tok
    res = llm.generate(prompts, [SamplingParams.greedy(12, stop=[stop, "never"], ignore_eos=True),
                                 SamplingParams.greedy(12, ignore_eos=True)])
    assert res[0].finish_reason == FinishReason.STOP
    assert res[0].text == text[:first]
    assert res[0].output_token_ids == free[:first + len(stop)]
    assert res[1].finish_reason == FinishReason.LENGTH and len(res[1].output_token_ids) == 12
    assert res[1].text == tok.decode(res[1].output_token_ids)
    st = llm.engine.runner.cache.stats()
    assert st.num_free == st.num_pages and st.num_sequences == 0


def test_scratch_guards_catch_a_write_outside_a_buffer():
    """The debugging arena: guard elements around every buffer keep their pattern unless
    something writes outside the buffer it was given."""
    from emberserve_b200.engine.runner import ScratchArena

    arena = ScratchArena(torch.device("cpu"), guard=8)
    a = arena("a", (3, 5), torch.float32)
    b = arena("b", (7,), torch.bfloat16)
    a.fill_(1.0)
    b.fill_(2.0)
    arena.verify()
    assert a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0
    grown = arena("a", (4, 5), torch.float32)  # a larger request replaces the buffer, guards and all
    grown.zero_()
    arena.verify()
    flat = grown.view(-1)
    torch.as_strided(flat, (1,), (1,), storage_offset=flat.storage_offset() + flat.numel())[0] = 3.0
    with pytest.raises(RuntimeError, match="wrote after"):
        arena.verify()
    plain_arena = ScratchArena(torch.device("cpu"))
    plain_arena("x", (4,), torch.float32)
    plain_arena.verify()  # nothing to check without guards


def test_step_trace_file(model_dirs, tmp_path, monkeypatch):
    """EMBERSERVE_STEP_TRACE=path: one JSON line of step statistics per step."""
    import json

    path = tmp_path / "steps.jsonl"
    monkeypatch.setenv("EMBERSERVE_STEP_TRACE", str(path))
    name = "tiny_a"
    llm = make_llm(model_dirs[name], name, max_num_batched_tokens=8)
    llm.generate(prompts_for(name, [11, 3]), SamplingParams.greedy(4, ignore_eos=True))
    lines = [json.loads(x) for x in path.read_text().splitlines()]
    assert len(lines) >= 4 and [x["step"] for x in lines] == sorted(x["step"] for x in lines)
    assert sum(x["num_prefill_tokens"] for x in lines) == 14
    assert sum(x["num_decode_tokens"] for x in lines) == 6
    assert all(x["num_tokens"] <= 8 for x in lines)
