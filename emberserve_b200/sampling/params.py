"""Per-request sampling parameters, with the reference's names, defaults and checks
(``emberserve/sched/request.py:14-40``)."""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class SamplingParams:
    max_tokens: int = 128
    temperature: float = 1.0  # 0.0 -> greedy
    top_k: int = -1  # -1 -> off
    top_p: float = 1.0  # 1.0 -> off
    repetition_penalty: float = 1.0  # 1.0 -> off; > 1 penalises tokens already in prompt + output
    stop_token_ids: list[int] = field(default_factory=list)
    stop: list[str] = field(default_factory=list)  # stop strings need a tokenizer
    ignore_eos: bool = False
    seed: int | None = None  # per-request seed for reproducible sampling
    logprobs: int | None = None  # reserved

    def __post_init__(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.temperature < 0.0:
            raise ValueError("temperature must be >= 0")
        if not (self.top_k == -1 or self.top_k >= 1):
            raise ValueError("top_k must be -1 or >= 1")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.repetition_penalty <= 0.0:
            raise ValueError("repetition_penalty must be > 0")

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0.0

    @classmethod
    def greedy(cls, max_tokens: int = 128, **kw) -> "SamplingParams":
        return cls(max_tokens=max_tokens, temperature=0.0, **kw)
