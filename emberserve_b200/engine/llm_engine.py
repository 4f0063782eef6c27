"""The engine: requests in, tokens out, one ``step()`` at a time.

``LLMEngine`` owns the model runner (weights, cache, kernels), the scheduler and the
sampler.  A step: schedule -> build the rows -> ``ModelRunner.step`` -> sample the rows
whose prompt is complete -> advance, stop-check, finish and free.

With ``EngineConfig.async_scheduling`` (the default) the last part trails by one step: a
call of ``step()`` schedules and launches step n and only then reads the tokens of step
n - 1, so the host's share of a step (scheduling, packing, bookkeeping) runs while the
device computes.  The sampled tokens stay on the device (``ModelRunner.token_feedback``)
and the rows of step n name them by index; on the host a placeholder stands in the
request's output until the token arrives.  A request that turns out to have ended with the
token of step n - 1 (an end-of-sequence token) has then already been given a row in step n:
that row's token is dropped and the pages go back when the end is seen.  The reference has
no such mode (``emberserve/engine.py:643-706`` reads every step's tokens before it plans
the next).  Names and meanings
follow ``emberserve/engine.py``: ``from_pretrained`` (``:383-426``), ``add_request``
(``:600-619``), ``step`` (``:643-706``), ``abort_request``, ``has_unfinished_requests``,
``reset``; ``StepStats`` (``:46-61``) and the per-request metrics (``:1089-1099``).
"""

from __future__ import annotations

import contextlib
import dataclasses
import json
import os
import time
from dataclasses import dataclass, field

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.config.engine import EngineConfig
from emberserve_b200.config.model import ModelConfig
from emberserve_b200.engine.detokenizer import Detokenizer
from emberserve_b200.tokenizer import load_tokenizer
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


@dataclass
class _InFlight:
    """A launched step whose tokens the host has not read yet."""

    requests: list[Request]  # the rows that sample, in order
    scheduled: list[Request]  # every request that had a row in the step
    places: list[int]  # where in each request's output its placeholder stands
    length_stop: list[bool]  # the token ends the request by count, whatever it is
    host: torch.Tensor | None  # pinned int32 copy of the tokens, valid after `event`
    event: "torch.cuda.Event | None"
    tokens: list[int] = field(default_factory=list)  # off the GPU: already on the host


class LLMEngine:
    def __init__(self, runner: ModelRunner, config: EngineConfig, tokenizer=None) -> None:
        self.runner = runner
        self.config = config
        self.model_config: ModelConfig = runner.config
        self.tokenizer = tokenizer
        self.detokenizer = Detokenizer(tokenizer)
        self.scheduler = Scheduler(config, runner.cache)
        self.sampler = Sampler(runner.device, seed=config.seed)
        # every id that ends a request: the configuration's, and the tokenizer's own end-of-sequence
        # id where there is a tokenizer (emberserve/engine.py:220-222)
        eos = set(getattr(self.model_config, "eos_token_ids", ()))
        if getattr(tokenizer, "eos_token_id", None) is not None:
            eos.add(int(tokenizer.eos_token_id))
        self.eos_token_ids = frozenset(eos)
        self._next_seq_id = 0
        self._step_count = 0
        self.keep_stats = False
        self.stats: list[StepStats] = []
        self._inflight: _InFlight | None = None
        self._final_text: dict[str, str] = {}  # text of the requests that ended last, until asked for
        # EMBERSERVE_STEP_TRACE=path: a line of step statistics per step is appended to that file
        # (the reference's switch of the same name, emberserve/steptrace.py:94-101)
        trace_path = os.environ.get("EMBERSERVE_STEP_TRACE")
        self._trace_file = open(trace_path, "a") if trace_path else None
        self._penalties_seen = False
        self._token_host: list[torch.Tensor | None] = [None, None]
        self._token_turn = 0
        runner.attn_kernel = config.attn_backend
        if config.max_num_seqs > runner.token_feedback.numel():
            raise ValueError(f"max_num_seqs={config.max_num_seqs} exceeds the {runner.token_feedback.numel()} "
                             f"sampled tokens a step may leave on the device for the next one")
        if config.enable_cuda_graphs:
            with self._on_device():
                runner.enable_graphs(config.max_model_len, config.max_num_seqs)
                if config.eager_graph_capture and runner.graphs is not None:
                    runner.graphs.capture_all()

    def _on_device(self):
        """The runner's GPU made the current device for what the engine launches itself (graph
        capture, the sampler, events): the kernels launch on the current device's stream."""
        if self.runner.device.type == "cuda":
            return torch.cuda.device(self.runner.device)
        return contextlib.nullcontext()

    @classmethod
    def from_pretrained(cls, model_dir: str | os.PathLike, engine_config: EngineConfig | None = None,
                        **overrides) -> "LLMEngine":
        unknown = [k for k in overrides if k not in {f.name for f in dataclasses.fields(EngineConfig)}]
        if unknown:
            raise TypeError(f"EngineConfig has no field {unknown[0]!r}")
        # a copy with the overrides: the caller's object is left as it is (replace() validates again)
        cfg = dataclasses.replace(engine_config or EngineConfig(), **overrides, model_dir=str(model_dir))
        runner = ModelRunner.from_dir(model_dir, cfg.dtype, device=cfg.device, **cls.runner_options(cfg))
        return cls(runner, cfg, tokenizer=load_tokenizer(model_dir))

    @staticmethod
    def runner_options(cfg: EngineConfig) -> dict:
        """What the model runner is built with under `cfg`: the page size and count, and the sizes
        of the largest steps, for which memory is kept free when the cache is sized from free
        memory (``emberserve/engine.py:121-139``: without chunked prefill a preempted request
        comes back with its whole history in one step, up to max_model_len tokens)."""
        chunk = cfg.max_num_batched_tokens
        if not cfg.enable_chunked_prefill:
            chunk = max(chunk, cfg.max_model_len)
        # More pages than max_num_seqs requests of max_model_len tokens can never be used.
        useful = cfg.max_num_seqs * (-(-cfg.max_model_len // cfg.block_size))
        return dict(page_size=cfg.block_size, num_pages=cfg.num_gpu_blocks, max_pages=useful,
                    num_state_slots=cfg.max_num_seqs, gpu_memory_utilization=cfg.gpu_memory_utilization,
                    max_step_tokens=chunk, max_graph_rows=cfg.max_num_seqs if cfg.enable_cuda_graphs else 0,
                    max_logit_rows=cfg.max_num_seqs, scratch_guard=cfg.debug_scratch_guard,
                    tiled_weight_copies=cfg.tiled_weight_copies)

    @classmethod
    def from_runner(cls, runner: ModelRunner, engine_config: EngineConfig | None = None) -> "LLMEngine":
        cfg = engine_config or EngineConfig(dtype=runner.dtype, block_size=runner.page_size)
        return cls(runner, cfg)

    # ---- convenience ------------------------------------------------------------------------
    FINAL_TEXT_KEEP = 1024

    def _keep_final_text(self, request_id: str) -> None:
        if self.tokenizer is not None:
            self._final_text[request_id] = self.detokenizer.text(request_id)
            while len(self._final_text) > self.FINAL_TEXT_KEEP:
                self._final_text.pop(next(iter(self._final_text)))
        self.detokenizer.drop(request_id)

    def output_text(self, request_id: str, take: bool = True) -> str:
        """Text so far of a live request, or the whole text of one that has ended (handed out once
        unless `take` is false; the last FINAL_TEXT_KEEP ended requests are kept;
        emberserve/engine.py:1102-1107)."""
        if request_id in self._final_text:
            return self._final_text.pop(request_id) if take else self._final_text[request_id]
        return self.detokenizer.text(request_id)

    def release_graphs(self) -> None:
        """Let go of the captured CUDA graphs; decode steps then launch their kernels one by one
        (emberserve/engine.py:564-573)."""
        import gc

        if self.runner.device.type == "cuda":
            torch.cuda.synchronize(self.runner.device)  # a step that was launched from a graph has run
        self.runner.use_graphs = False
        self.runner.graphs = None
        gc.collect()

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
        if req.sampling_params.repetition_penalty != 1.0:
            self._penalties_seen = True
        self._next_seq_id += 1
        self.scheduler.add_request(req)
        return req

    def abort_request(self, request_id: str) -> None:
        self.scheduler.abort_request(request_id)
        self.detokenizer.drop(request_id)

    def has_unfinished_requests(self) -> bool:
        # (a launched step whose tokens are still to be read belongs to requests that are
        # running or waiting, unless they were aborted since)
        return self.scheduler.has_unfinished_requests()

    def reset(self) -> None:
        self._inflight = None
        self._final_text.clear()
        for req in list(self.scheduler.running) + list(self.scheduler.waiting):
            self.scheduler.abort_request(req.request_id)
            self.detokenizer.drop(req.request_id)
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
        """One step.  With async scheduling the outputs are those of the step launched by the
        call before this one; a last call with nothing left to launch returns the rest."""
        if not self.config.async_scheduling or self._history_needed():
            outputs = self._finalize(self._take_inflight())
            outputs += self._step_sync()
            self.runner.verify_scratch()
            return outputs
        so = self.scheduler.schedule()
        if so.is_empty:
            if self._inflight is None:
                return self._drop_stuck()
            return self._finalize(self._take_inflight())
        before = self._take_inflight()
        self._inflight = self._launch(so)
        self.runner.verify_scratch()  # (does nothing unless the scratch buffers are guarded)
        return self._finalize(before)

    def drain(self):
        """Run steps until no request is left; yields the final ``RequestOutput`` of each request
        as it ends (its text is then to be had from ``output_text``)."""
        while self.has_unfinished_requests():
            for out in self.step():
                if out.finished:
                    yield out

    def _history_needed(self) -> bool:
        """Whether some live request samples with its token history (kept on the host)."""
        if not self._penalties_seen:
            return False
        live = list(self.scheduler.running) + list(self.scheduler.waiting)
        if any(r.sampling_params.repetition_penalty != 1.0 for r in live):
            return True
        self._penalties_seen = False
        return False

    def _take_inflight(self) -> "_InFlight | None":
        inflight, self._inflight = self._inflight, None
        return inflight

    def _drop_stuck(self) -> list[RequestOutput]:
        """Nothing could be scheduled, nothing runs and nothing is on its way, yet a request
        waits: with the whole cache free it still does not fit (a request that outgrew the pool
        and preempted itself), so it never will.  It ends with ABORT and what it has produced
        (the reference's server loop does the same, ``emberserve/server/engine_core.py:246-254``)."""
        if self.scheduler.running or not self.scheduler.waiting:
            return []
        req = self.scheduler.waiting[0]
        self.scheduler.finish_request(req, FinishReason.ABORT)
        return [RequestOutput(request_id=req.request_id, new_token_ids=[],
                              output_token_ids=list(req.output_token_ids), finished=True,
                              finish_reason=FinishReason.ABORT, metrics=self._metrics(req))]

    def _step_sync(self) -> list[RequestOutput]:
        so = self.scheduler.schedule()
        if so.is_empty:
            return self._drop_stuck()
        self._step_count += 1
        t0 = time.perf_counter()
        logits = self.runner.step(self.build_rows(so))
        t1 = time.perf_counter()
        sampling = [r for r, done in zip(so.scheduled, so.prefill_complete) if done]
        with self._on_device():
            tokens = self.sampler.sample(logits, sampling) if sampling else []  # (reading them waits for the step)
        t2 = time.perf_counter()
        for req, qlen in zip(so.scheduled, so.query_lens):
            req.num_computed_tokens += qlen
        if sampling:
            self._check_kernels(so.scheduled)
        outputs = self._postprocess(sampling, tokens)
        self._record(so, (t1 - t0) * 1e3, (t2 - t1) * 1e3)
        return outputs

    def _check_kernels(self, scheduled: list[Request]) -> None:
        """Called once the host has waited for a step: if a bounded wait inside one of the
        tcgen05 kernels ran out, what the step computed is invalid (its logits, and the keys and
        values it cached).  No token of it is handed out: the step's requests, and those of a step
        launched behind it from its tokens, end with ABORT, their pages go back, the status word is
        cleared and the error is raised."""
        try:
            K.check_status()
        except K.KernelError:
            behind, self._inflight = self._inflight, None
            for req in list(scheduled) + (list(behind.scheduled) if behind is not None else []):
                if not req.is_finished:
                    req.hold = False
                    while req.output_token_ids and req.output_token_ids[-1] < 0:
                        req.output_token_ids.pop()  # placeholders of tokens that never arrive
                    self.scheduler.finish_request(req, FinishReason.ABORT)
                    self.detokenizer.drop(req.request_id)
            raise

    def _record(self, so: SchedulerOutput, forward_ms: float, sample_ms: float) -> None:
        if not self.keep_stats and self._trace_file is None:
            return
        st = StepStats(
            step=self._step_count, is_prefill=so.is_prefill, num_seqs=len(so.scheduled),
            num_tokens=so.num_tokens, num_preempted=len(so.preempted),
            forward_ms=forward_ms, sample_ms=sample_ms,
            num_free_pages=self.runner.cache.num_free_pages(0) if self.runner.cache.pools else 0,
            num_prefill_tokens=so.num_prefill_tokens, num_decode_tokens=so.num_decode_tokens)
        if self.keep_stats:
            self.stats.append(st)
        if self._trace_file is not None:  # one JSON line per step (emberserve/steptrace.py:48-76)
            self._trace_file.write(json.dumps(dict(dataclasses.asdict(st), t=time.time(),
                                                   async_scheduling=self.config.async_scheduling)) + "\n")
            self._trace_file.flush()

    def _launch(self, so: SchedulerOutput) -> _InFlight:
        """Run the step and sample on the device; nothing here waits for the device.  The
        times in the step's StepStats are therefore those of the launches."""
        self._step_count += 1
        t0 = time.perf_counter()
        logits = self.runner.step(self.build_rows(so))
        t1 = time.perf_counter()
        sampling = [r for r, done in zip(so.scheduled, so.prefill_complete) if done]
        host = event = None
        tokens: list[int] = []
        if sampling:
            n = len(sampling)
            with self._on_device():
                dev_tokens = self.sampler.sample_tensor(logits, sampling, out=self.runner.token_feedback[:n])
                if dev_tokens.is_cuda:
                    turn = self._token_turn
                    self._token_turn ^= 1
                    if self._token_host[turn] is None or self._token_host[turn].numel() < n:
                        self._token_host[turn] = torch.empty(max(n, 256), dtype=torch.int32, pin_memory=True)
                    host = self._token_host[turn]
                    host[:n].copy_(dev_tokens, non_blocking=True)
                    event = K.record_event()
                else:
                    tokens = dev_tokens.tolist()
        t2 = time.perf_counter()
        for req, qlen in zip(so.scheduled, so.query_lens):
            req.num_computed_tokens += qlen
        places, length_stop = [], []
        for k, req in enumerate(sampling):
            req.append_output(-(k + 1))  # stands for token_feedback[k] until the token is read
            places.append(req.num_output_tokens - 1)
            by_count = (req.num_output_tokens >= req.sampling_params.max_tokens
                        or req.num_tokens >= self.config.max_model_len)
            length_stop.append(by_count)
            req.hold = by_count
        self._record(so, (t1 - t0) * 1e3, (t2 - t1) * 1e3)
        return _InFlight(sampling, list(so.scheduled), places, length_stop, host, event, tokens)

    def _finalize(self, inflight: "_InFlight | None") -> list[RequestOutput]:
        """Read the tokens of a launched step and do what follows from them."""
        if inflight is None or not inflight.requests:
            return []
        if inflight.event is not None:
            inflight.event.synchronize()
        self._check_kernels(inflight.scheduled)  # the step has run: did all of its kernels?
        if inflight.event is not None:
            tokens = inflight.host[:len(inflight.requests)].tolist()
        else:
            tokens = inflight.tokens
        now = time.perf_counter()
        outputs = []
        for req, place, by_count, tok in zip(inflight.requests, inflight.places, inflight.length_stop,
                                             tokens, strict=True):
            if req.is_finished:  # aborted, or ended by an earlier token while this one was on its way
                continue
            req.output_token_ids[place] = int(tok)
            if req.first_token_time is None:
                req.first_token_time = now
            params = req.sampling_params
            reason = None
            if (tok in self.eos_token_ids and not params.ignore_eos) or tok in params.stop_token_ids:
                reason = FinishReason.STOP
            elif by_count:
                reason = FinishReason.LENGTH
            text, matched = self.detokenizer.feed(req.request_id, req.output_token_ids[:place + 1], params.stop,
                                                  final=reason is not None)
            if matched is not None and reason is None:
                reason = FinishReason.STOP  # the text has reached a stop string
            if reason is not None:
                del req.output_token_ids[place + 1:]  # a placeholder of the step launched since
                req.hold = False
                self.scheduler.finish_request(req, reason)
                self._keep_final_text(req.request_id)
            outputs.append(RequestOutput(
                request_id=req.request_id, new_token_ids=[int(tok)],
                output_token_ids=req.output_token_ids[:place + 1], finished=reason is not None,
                finish_reason=reason, text_delta=text,
                metrics=self._metrics(req) if reason is not None else {}))
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
            text, matched = self.detokenizer.feed(req.request_id, req.output_token_ids, req.sampling_params.stop,
                                                  final=reason is not None)
            if matched is not None and reason is None:
                reason = FinishReason.STOP  # the text has reached a stop string
            if reason is not None:
                self.scheduler.finish_request(req, reason)
                self._keep_final_text(req.request_id)
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
