"""The engine: requests in, tokens out, one ``step()`` at a time.

``LLMEngine`` owns the model runner (weights, cache, kernels), the scheduler and the
sampler.  A step: schedule -> build the rows -> ``ModelRunner.step`` -> sample the rows
whose prompt is complete -> advance, stop-check, finish and free.  Names and meanings
follow ``emberserve/engine.py``: ``from_pretrained`` (``:383-426``), ``add_request``
(``:600-619``), ``step`` (``:643-706``), ``abort_request``, ``has_unfinished_requests``,
``reset``; ``StepStats`` (``:46-61``) and the per-request metrics (``:1089-1099``).
"""

from __future__ import annotations

import os
import time
from dataclasses import dataclass

import torch

from emberserve_b200.config.engine import EngineConfig
from emberserve_b200.config.model import ModelConfig
from emberserve_b200.engine.request import (FinishReason, Request, RequestOutput, check_stop)
from emberserve_b200.engine.runner import ModelRunner, StepRow
from emberserve_b200.engine.scheduler import Scheduler, SchedulerOutput
from emberserve_b200.sampling.params import SamplingParams
from emberserve_b200.sampling.sampler import Sampler


@dataclass
class StepStats:
    step: int
    is_prefill: bool
    num_seqs: int
    num_tokens: int
    num_preempted: int
    forward_ms: float
    sample_ms: float
    num_free_pages: int
    num_prefill_tokens: int
    num_decode_tokens: int


class LLMEngine:
    def __init__(self, runner: ModelRunner, config: EngineConfig, tokenizer=None) -> None:
        self.runner = runner
        self.config = config
        self.model_config: ModelConfig = runner.config
        self.tokenizer = tokenizer
        self.scheduler = Scheduler(config, runner.cache)
        self.sampler = Sampler(runner.device)
        self.eos_token_ids = frozenset(getattr(self.model_config, "eos_token_ids", ()))
        self._next_seq_id = 0
        self._step_count = 0
        self.keep_stats = False
        self.stats: list[StepStats] = []
        if config.enable_cuda_graphs:
            runner.enable_graphs(config.max_model_len, config.max_num_seqs)

    @classmethod
    def from_pretrained(cls, model_dir: str | os.PathLike, engine_config: EngineConfig | None = None,
                        **overrides) -> "LLMEngine":
        cfg = engine_config or EngineConfig()
        for key, value in overrides.items():
            if not hasattr(cfg, key):
                raise TypeError(f"EngineConfig has no field {key!r}")
            setattr(cfg, key, value)
        cfg.__post_init__()
        cfg.model_dir = str(model_dir)
        # More pages than max_num_seqs requests of max_model_len tokens can never be used.
        useful = cfg.max_num_seqs * (-(-cfg.max_model_len // cfg.block_size))
        runner = ModelRunner.from_dir(
            model_dir, cfg.dtype, device=cfg.device, page_size=cfg.block_size,
            num_pages=cfg.num_gpu_blocks, max_pages=useful, num_state_slots=cfg.max_num_seqs,
            gpu_memory_utilization=cfg.gpu_memory_utilization)
        return cls(runner, cfg, tokenizer=_load_tokenizer(model_dir))

    @classmethod
    def from_runner(cls, runner: ModelRunner, engine_config: EngineConfig | None = None) -> "LLMEngine":
        cfg = engine_config or EngineConfig(dtype=runner.dtype, block_size=runner.page_size)
        return cls(runner, cfg)

    # ---- requests --------------------------------------------------------------------------
    def add_request(self, request_id: str, prompt: str | list[int],
                    sampling_params: SamplingParams | None = None, arrival_time: float | None = None,
                    metadata: dict | None = None) -> Request:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("engine has no tokenizer; pass prompt token ids")
            prompt_ids = list(self.tokenizer.encode(prompt))
        else:
            prompt_ids = [int(t) for t in prompt]
        if prompt_ids and (max(prompt_ids) >= self.runner.vocab_size or min(prompt_ids) < 0):
            raise ValueError(f"prompt token id out of vocabulary (vocab_size {self.runner.vocab_size})")
        req = Request(request_id=request_id, prompt_token_ids=prompt_ids,
                      sampling_params=sampling_params or SamplingParams(),
                      seq_id=self._next_seq_id, metadata=dict(metadata or {}))
        if arrival_time is not None:
            req.arrival_time = arrival_time
        self._next_seq_id += 1
        self.scheduler.add_request(req)
        return req

    def abort_request(self, request_id: str) -> None:
        self.scheduler.abort_request(request_id)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished_requests()

    def reset(self) -> None:
        for req in list(self.scheduler.running) + list(self.scheduler.waiting):
            self.scheduler.abort_request(req.request_id)
        self.runner.cache.reset()
        self.stats.clear()

    # ---- the step ----------------------------------------------------------------------------
    def build_rows(self, so: SchedulerOutput, all_positions: bool = False) -> list[StepRow]:
        rows = []
        for req, qlen, done in zip(so.scheduled, so.query_lens, so.prefill_complete):
            start = req.num_computed_tokens
            want = list(range(qlen)) if all_positions else ([qlen - 1] if done else [])
            rows.append(StepRow(req.seq_id, req.tokens_between(start, start + qlen), start, want))
        return rows

    def step_logits(self, so: SchedulerOutput, all_positions: bool = False) -> torch.Tensor:
        """Logits of a scheduled step without sampling or bookkeeping
        (``emberserve/engine.py:883-900``); the cache is written as in a real step."""
        logits = self.runner.step(self.build_rows(so, all_positions))
        for req, qlen in zip(so.scheduled, so.query_lens):
            req.num_computed_tokens += qlen
        return logits

    def step(self) -> list[RequestOutput]:
        so = self.scheduler.schedule()
        if so.is_empty:
            return []
        self._step_count += 1
        t0 = time.perf_counter()
        logits = self.runner.step(self.build_rows(so))
        t1 = time.perf_counter()
        sampling = [r for r, done in zip(so.scheduled, so.prefill_complete) if done]
        tokens = self.sampler.sample(logits, sampling) if sampling else []
        t2 = time.perf_counter()
        for req, qlen in zip(so.scheduled, so.query_lens):
            req.num_computed_tokens += qlen
        outputs = self._postprocess(sampling, tokens)
        if self.keep_stats:
            self.stats.append(StepStats(
                step=self._step_count, is_prefill=so.is_prefill, num_seqs=len(so.scheduled),
                num_tokens=so.num_tokens, num_preempted=len(so.preempted),
                forward_ms=(t1 - t0) * 1e3, sample_ms=(t2 - t1) * 1e3,
                num_free_pages=self.runner.cache.num_free_pages(0) if self.runner.cache.pools else 0,
                num_prefill_tokens=so.num_prefill_tokens, num_decode_tokens=so.num_decode_tokens))
        return outputs

    def _postprocess(self, requests: list[Request], tokens: list[int]) -> list[RequestOutput]:
        now = time.perf_counter()
        outputs = []
        for req, tok in zip(requests, tokens, strict=True):
            if req.is_finished:
                continue
            req.append_output(int(tok))
            if req.first_token_time is None:
                req.first_token_time = now
            reason = check_stop(req, int(tok), self.eos_token_ids, self.config.max_model_len)
            text = ""
            if self.tokenizer is not None:
                text = self.tokenizer.decode([int(tok)])
            if reason is not None:
                self.scheduler.finish_request(req, reason)
            outputs.append(RequestOutput(
                request_id=req.request_id, new_token_ids=[int(tok)],
                output_token_ids=list(req.output_token_ids), finished=reason is not None,
                finish_reason=reason, text_delta=text,
                metrics=self._metrics(req) if reason is not None else {}))
        return outputs

    @staticmethod
    def _metrics(req: Request) -> dict:
        m = {"num_prompt_tokens": req.num_prompt_tokens, "num_output_tokens": req.num_output_tokens}
        if req.first_token_time and req.arrival_time:
            m["ttft_s"] = req.first_token_time - req.arrival_time
        if req.finished_time and req.first_token_time and req.num_output_tokens > 1:
            m["tpot_s"] = (req.finished_time - req.first_token_time) / (req.num_output_tokens - 1)
        if req.finished_time and req.arrival_time:
            m["e2e_s"] = req.finished_time - req.arrival_time
        return m


def _load_tokenizer(model_dir):
    """A tokenizer, if the folder has one and a tokenizer library is installed; the engine
    itself works on token ids and needs none."""
    from pathlib import Path

    if not (Path(model_dir) / "tokenizer.json").is_file():
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    tok = Tokenizer.from_file(str(Path(model_dir) / "tokenizer.json"))

    class _Wrapper:
        def encode(self, text: str) -> list[int]:
            return tok.encode(text).ids

        def decode(self, ids: list[int]) -> str:
            return tok.decode(ids)

    return _Wrapper()
