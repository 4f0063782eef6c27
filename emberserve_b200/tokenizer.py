"""Text in, token ids out, and a conversation rendered through the model's chat template.

The engine works on token ids; text needs a ``tokenizer.json`` in the model folder (read with
the ``tokenizers`` library alone).  ``emberserve/tokenizer.py:20-67`` is the reference's wrapper
(it goes through ``transformers``): the same four operations, ``encode``, ``decode``,
``decode_batch`` and ``apply_chat_template``, and the tokenizer's own end-of-sequence id, which
the engine adds to the ids that end a request (``emberserve/engine.py:220-222``).

The chat template is the Jinja text that the model folder carries (``chat_template`` in
``tokenizer_config.json``, or a ``chat_template.jinja`` file); it is rendered with ``messages``,
``add_generation_prompt``, ``bos_token`` and ``eos_token`` in a sandboxed environment and the
result is encoded without further special tokens.  A folder without a template gets the ChatML
layout that Qwen2.5 uses: ``<|im_start|>role\\ncontent<|im_end|>\\n`` per message and
``<|im_start|>assistant\\n`` to open the reply.
"""

from __future__ import annotations

import json
from pathlib import Path


def has_tokenizer(model_dir: str | Path) -> bool:
    return (Path(model_dir) / "tokenizer.json").is_file()


def _token_text(entry) -> str | None:
    """``eos_token`` / ``bos_token`` of tokenizer_config.json: a string or {"content": ...}."""
    if isinstance(entry, str):
        return entry
    if isinstance(entry, dict) and isinstance(entry.get("content"), str):
        return entry["content"]
    return None


def chatml(messages: list[dict], add_generation_prompt: bool = True) -> str:
    text = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in messages)
    return text + ("<|im_start|>assistant\n" if add_generation_prompt else "")


class Tokenizer:
    def __init__(self, model_dir: str | Path) -> None:
        try:
            from tokenizers import Tokenizer as _Fast
        except ImportError as e:  # pragma: no cover
            raise ImportError("text prompts need the `tokenizers` package") from e
        d = Path(model_dir)
        self._tok = _Fast.from_file(str(d / "tokenizer.json"))
        cfg = {}
        if (d / "tokenizer_config.json").is_file():
            cfg = json.loads((d / "tokenizer_config.json").read_text())
        self.bos_token = _token_text(cfg.get("bos_token"))
        self.eos_token = _token_text(cfg.get("eos_token"))
        self.eos_token_id: int | None = None
        if self.eos_token is not None:
            self.eos_token_id = self._tok.token_to_id(self.eos_token)
        self.chat_template: str | None = None
        if (d / "chat_template.jinja").is_file():
            self.chat_template = (d / "chat_template.jinja").read_text()
        elif isinstance(cfg.get("chat_template"), str):
            self.chat_template = cfg["chat_template"]
        self._compiled = None

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        return list(self._tok.encode(text, add_special_tokens=add_special_tokens).ids)

    def decode(self, ids: list[int], skip_special_tokens: bool = False) -> str:
        return self._tok.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def decode_batch(self, batch: list[list[int]], skip_special_tokens: bool = False) -> list[str]:
        return self._tok.decode_batch([list(ids) for ids in batch], skip_special_tokens=skip_special_tokens)

    def render_chat(self, messages: list[dict], add_generation_prompt: bool = True) -> str:
        """The conversation as the text the model was trained on."""
        for m in messages:
            if not isinstance(m, dict) or "role" not in m or "content" not in m:
                raise ValueError("a message is a dict with 'role' and 'content'")
        if self.chat_template is None:
            return chatml(messages, add_generation_prompt)
        if self._compiled is None:
            from jinja2.sandbox import ImmutableSandboxedEnvironment

            def raise_exception(message: str):
                raise ValueError(f"chat template: {message}")

            env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
            env.globals["raise_exception"] = raise_exception
            self._compiled = env.from_string(self.chat_template)
        return self._compiled.render(messages=messages, add_generation_prompt=add_generation_prompt,
                                     bos_token=self.bos_token or "", eos_token=self.eos_token or "", tools=None)

    def apply_chat_template(self, messages: list[dict], add_generation_prompt: bool = True) -> list[int]:
        # the template writes its own special tokens as text; none are added on top
        return self.encode(self.render_chat(messages, add_generation_prompt), add_special_tokens=False)


def load_tokenizer(model_dir: str | Path) -> Tokenizer | None:
    """A tokenizer, if the folder has one and the ``tokenizers`` library is installed."""
    if not has_tokenizer(model_dir):
        return None
    try:
        import tokenizers  # noqa: F401
    except ImportError:
        return None
    return Tokenizer(model_dir)
