"""Request life-cycle types.

The SCHEMA here is the reference's, kept on purpose so that its users find what they know:
the states, the finish reasons, and the fields and small accessors of ``Request`` and
``RequestOutput`` are those of ``emberserve/sched/request.py:43-138``, name for name.  This
engine's own are ``hold`` (asynchronous stepping), ``tokens_between`` (the step function takes
tokens, not requests) and ``check_stop`` living here rather than beside the sampler.

A request moves WAITING -> RUNNING -> FINISHED, or back to the front of the waiting queue
when it is preempted: it keeps its generated tokens and recomputes everything.  Token ids
are the source of truth; ``num_computed_tokens`` is the request's position in the cache.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from enum import Enum

from emberserve_b200.sampling.params import SamplingParams


class RequestState(str, Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED = "finished"


class FinishReason(str, Enum):
    STOP = "stop"  # eos or a stop token
    LENGTH = "length"  # max_tokens or the model length limit
    ABORT = "abort"


@dataclass
class Request:
    request_id: str
    prompt_token_ids: list[int]
    sampling_params: SamplingParams
    # -- where it stands ------------------------------------------------------------------
    state: RequestState = RequestState.WAITING
    finish_reason: FinishReason | None = None
    seq_id: int = -1  # integer id used by the cache manager; assigned by the engine
    num_computed_tokens: int = 0  # its position in the cache
    output_token_ids: list[int] = field(default_factory=list)
    # Set while the request's last token is still on its way from the device and is known to end
    # it (max_tokens or the model length): the scheduler gives it no further token.
    hold: bool = False
    # -- clock readings (time.perf_counter) for the metrics of its final output ---------------
    arrival_time: float = field(default_factory=time.perf_counter)
    first_scheduled_time: float | None = None
    first_token_time: float | None = None
    finished_time: float | None = None
    metadata: dict = field(default_factory=dict)

    @property
    def is_finished(self) -> bool:
        return self.state == RequestState.FINISHED

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self.output_token_ids)

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    def tokens_between(self, start: int, end: int) -> list[int]:
        """Tokens [start, end) of prompt + output: what a step that computes these positions is fed."""
        n = len(self.prompt_token_ids)
        if end <= n:
            return self.prompt_token_ids[start:end]
        if start >= n:
            return self.output_token_ids[start - n:end - n]
        return self.prompt_token_ids[start:] + self.output_token_ids[:end - n]

    def append_output(self, token_id: int) -> None:
        self.output_token_ids.append(token_id)

    def reset_for_recompute(self) -> None:
        """Preemption by recompute: keep the generated tokens, drop the cache position
        (``request.py:120-124``)."""
        self.state = RequestState.PREEMPTED
        self.num_computed_tokens = 0


@dataclass
class RequestOutput:
    """What a step yields for a request that produced a token or finished."""

    request_id: str
    new_token_ids: list[int]
    output_token_ids: list[int]
    finished: bool
    finish_reason: FinishReason | None = None
    text_delta: str = ""
    metrics: dict = field(default_factory=dict)


def check_stop(request: Request, token_id: int, eos_token_ids, max_model_len: int) -> FinishReason | None:
    """Whether `request` is done, AFTER `token_id` was appended.  eos (unless ignore_eos)
    or a stop token -> STOP; max_tokens or the model length -> LENGTH; STOP wins
    (``emberserve/sampling.py:148-164``)."""
    params = request.sampling_params
    if token_id in eos_token_ids and not params.ignore_eos:
        return FinishReason.STOP
    if token_id in params.stop_token_ids:
        return FinishReason.STOP
    if request.num_output_tokens >= params.max_tokens or request.num_tokens >= max_model_len:
        return FinishReason.LENGTH
    return None
