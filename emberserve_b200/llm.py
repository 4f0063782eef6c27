"""The offline entry point: ``LLM(model_dir).generate(prompts, sampling_params)``.

The surface is the reference's (``emberserve/llm.py:13-64``): the constructor takes a model
folder, an ``EngineConfig`` and overrides of its fields; ``generate`` takes text or token-id
prompts with one ``SamplingParams`` for all or one per prompt, names the requests ``req-0``,
``req-1``, ... and returns one ``GenerationResult`` per prompt, in the order of the prompts;
``chat`` renders conversations through the model's chat template first.  The work itself is
the engine's: requests are submitted, ``LLMEngine.drain()`` runs steps until none is left and
hands over each request as it ends, and the text comes from the engine's detokenizer.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Sequence

from emberserve_b200.config.engine import EngineConfig
from emberserve_b200.engine.llm_engine import LLMEngine
from emberserve_b200.engine.request import FinishReason
from emberserve_b200.sampling.params import SamplingParams

Params = SamplingParams | Sequence[SamplingParams] | None


@dataclass
class GenerationResult:
    request_id: str
    prompt_token_ids: list[int]
    output_token_ids: list[int]
    text: str
    finish_reason: FinishReason | None
    metrics: dict = field(default_factory=dict)


def _one_per_prompt(count: int, given: Params) -> list[SamplingParams]:
    if given is None:
        given = SamplingParams()
    if isinstance(given, SamplingParams):
        return [given] * count
    given = list(given)
    if len(given) != count:
        raise ValueError(f"{len(given)} SamplingParams for {count} prompts: pass one for all, or one per prompt")
    return given


class LLM:
    def __init__(self, model_dir: str | Path | None = None, engine_config: EngineConfig | None = None, *,
                 engine: LLMEngine | None = None, **overrides) -> None:
        """Load `model_dir` into a new engine, or (``engine=``) wrap one that exists."""
        if (engine is None) == (model_dir is None):
            raise ValueError("give either a model folder or an engine")
        self.engine = engine if engine is not None else LLMEngine.from_pretrained(model_dir, engine_config, **overrides)

    @classmethod
    def from_engine(cls, engine: LLMEngine) -> "LLM":
        return cls(engine=engine)

    def generate(self, prompts: Sequence[str] | Sequence[list[int]], sampling_params: Params = None,
                 ) -> list[GenerationResult]:
        engine = self.engine
        submitted = {}
        for index, (prompt, params) in enumerate(zip(prompts, _one_per_prompt(len(prompts), sampling_params))):
            request = engine.add_request(f"req-{index}", prompt, params)
            submitted[request.request_id] = request
        ended: dict[str, GenerationResult] = {}
        for last in engine.drain():
            request = submitted.get(last.request_id)
            if request is None:  # a request that somebody else gave the engine
                continue
            ended[last.request_id] = GenerationResult(
                request_id=last.request_id, prompt_token_ids=request.prompt_token_ids,
                output_token_ids=last.output_token_ids, text=engine.output_text(last.request_id, take=False),
                finish_reason=last.finish_reason, metrics=last.metrics)
        return [ended[request_id] for request_id in submitted]

    def chat(self, conversations: Sequence[list[dict]], sampling_params: Params = None) -> list[GenerationResult]:
        """One reply per conversation (a list of {"role", "content"} messages), rendered through
        the chat template of the model folder (``emberserve/llm.py:59-64``)."""
        render = getattr(self.engine.tokenizer, "apply_chat_template", None)
        if render is None:
            raise ValueError("chat() needs a tokenizer with a chat template in the model folder")
        return self.generate([render(messages) for messages in conversations], sampling_params)
