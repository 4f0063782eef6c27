"""Offline batch entry point: ``LLM(model_dir).generate(prompts, sampling_params)``
(``emberserve/llm.py:13-64``: same constructor, same ``generate`` contract, request ids
``req-{i}``, results in the order of the prompts)."""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path

from emberserve_b200.config.engine import EngineConfig
from emberserve_b200.engine.llm_engine import LLMEngine
from emberserve_b200.engine.request import FinishReason, RequestOutput
from emberserve_b200.sampling.params import SamplingParams


@dataclass
class GenerationResult:
    request_id: str
    prompt_token_ids: list[int]
    output_token_ids: list[int]
    text: str
    finish_reason: FinishReason | None
    metrics: dict = field(default_factory=dict)


class LLM:
    def __init__(self, model_dir: str | Path, engine_config: EngineConfig | None = None,
                 **overrides) -> None:
        self.engine = LLMEngine.from_pretrained(model_dir, engine_config, **overrides)

    @classmethod
    def from_engine(cls, engine: LLMEngine) -> "LLM":
        obj = cls.__new__(cls)
        obj.engine = engine
        return obj

    def chat(self, conversations: list[list[dict]],
             sampling_params: SamplingParams | list[SamplingParams] | None = None) -> list[GenerationResult]:
        """One reply per conversation (a list of {"role", "content"} messages), rendered through the
        model's chat template (emberserve/llm.py:59-64); needs a tokenizer."""
        tok = self.engine.tokenizer
        if tok is None or not hasattr(tok, "apply_chat_template"):
            raise ValueError("chat() needs a tokenizer")
        return self.generate([tok.apply_chat_template(msgs) for msgs in conversations], sampling_params)

    def generate(self, prompts: list[str] | list[list[int]],
                 sampling_params: SamplingParams | list[SamplingParams] | None = None,
                 ) -> list[GenerationResult]:
        params = sampling_params or SamplingParams()
        if not isinstance(params, list):
            params = [params] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        reqs = [self.engine.add_request(f"req-{i}", p, sp)
                for i, (p, sp) in enumerate(zip(prompts, params, strict=True))]
        text: dict[str, list[str]] = {r.request_id: [] for r in reqs}
        final: dict[str, RequestOutput] = {}
        while self.engine.has_unfinished_requests():
            for out in self.engine.step():
                text[out.request_id].append(out.text_delta)
                if out.finished:
                    final[out.request_id] = out
        results = []
        for r in reqs:
            out = final[r.request_id]
            results.append(GenerationResult(
                request_id=r.request_id, prompt_token_ids=r.prompt_token_ids,
                output_token_ids=out.output_token_ids, text="".join(text[r.request_id]),
                finish_reason=out.finish_reason, metrics=out.metrics))
        return results
