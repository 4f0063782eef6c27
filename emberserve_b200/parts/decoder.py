"""A decoder assembled from parts: embedding, blocks in a given order, final norm, head.

The *order* in which blocks run is data: a list of ``LayerCall``.  It may name a block
twice (the block's weights are then used at two depths, each call with a cache entry of
its own) and it may let a call read the cache entry that an earlier call wrote.  Qwen2 is
the plain case: call i runs block i and owns entry i
(``emberserve/model/qwen2.py:167-187``).

Logits come back in float32 for the wanted token rows only; the final norm and the head
run on those rows alone (``qwen2.py:214-225`` selects rows before the head too).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import (Block, CacheNeed, ParamSpec, Part, SharedParts, Source,
                                        StepContext, build_part)
from emberserve_b200.parts.linear import linear_f32_out


@dataclass(frozen=True)
class LayerCall:
    layer: int  # index into DecoderSpec.layers
    cache: int | None  # id of the cache entry this call uses; None = the block keeps nothing
    write: bool = True  # False: the call reads the entry another call wrote in this step


@dataclass
class DecoderSpec:
    vocab_size: int
    hidden: int
    embed_name: str  # checkpoint tensor [vocab, hidden]
    layers: list[Any]  # block specs
    order: list[LayerCall]
    final_norm: Any  # norm spec
    head_name: str | None  # checkpoint tensor [vocab, hidden]; None = tied to the embedding
    max_positions: int
    # Checkpoint tensors that may be present but are not parameters: exact names or
    # suffixes (``emberserve/model/weights.py:22`` skips rotary_emb.inv_freq).
    ignorable: tuple[str, ...] = ("rotary_emb.inv_freq",)
    embedding_position: Any | None = None


class Decoder:
    def __init__(self, spec: DecoderSpec) -> None:
        self.spec = spec
        self.shared = SharedParts()
        self.blocks: list[Block] = [
            build_part("block", b, f"layers.{i}", self.shared) for i, b in enumerate(spec.layers)]
        self.final_norm = build_part("norm", spec.final_norm, "final_norm", self.shared)
        self.embed_position = (self.shared.get("position", spec.embedding_position)
                               if spec.embedding_position is not None else None)
        self.embed: torch.Tensor | None = None
        self.head: torch.Tensor | None = None
        self._entries = self._check_order()

    # ---- structure -------------------------------------------------------------------
    def _check_order(self) -> list[CacheNeed]:
        spec = self.spec
        entries: dict[int, CacheNeed] = {}
        for pos, call in enumerate(spec.order):
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"order[{pos}] names layer {call.layer}, model has {len(self.blocks)}")
            need = self.blocks[call.layer].cache_need()
            if call.cache is None:
                if need is not None:
                    raise ValueError(f"order[{pos}]: layer {call.layer} needs a cache entry")
                continue
            if need is None:
                raise ValueError(f"order[{pos}]: layer {call.layer} keeps nothing but names entry {call.cache}")
            if call.write:
                if call.cache in entries:
                    raise ValueError(f"order[{pos}]: cache entry {call.cache} is written twice")
                entries[call.cache] = need
            else:
                if call.cache not in entries:
                    raise ValueError(f"order[{pos}]: reads cache entry {call.cache} before it is written")
                if entries[call.cache] != need:
                    raise ValueError(f"order[{pos}]: layer {call.layer} needs {need}, entry "
                                     f"{call.cache} holds {entries[call.cache]}")
        if sorted(entries) != list(range(len(entries))):
            raise ValueError(f"cache entry ids must be 0..n-1, got {sorted(entries)}")
        return [entries[i] for i in range(len(entries))]

    def cache_entries(self) -> list[CacheNeed]:
        """What each cache entry must hold, by entry id."""
        return list(self._entries)

    def _walk(self) -> list[tuple[str, Part]]:
        out: list[tuple[str, Part]] = []

        def rec(path: str, part: Part) -> None:
            out.append((path, part))
            for name, child in part.children().items():
                rec(f"{path}.{name}", child)

        for i, b in enumerate(self.blocks):
            rec(f"layers.{i}", b)
        rec("final_norm", self.final_norm)
        for j, p in enumerate(self.shared.all()):
            rec(f"shared.{j}", p)
        return out

    def param_table(self) -> dict[str, ParamSpec]:
        """Every parameter of the model: local path -> shape and checkpoint sources."""
        s = self.spec
        table: dict[str, ParamSpec] = {
            "embed": ParamSpec((s.vocab_size, s.hidden), [Source(s.embed_name)])}
        if s.head_name is not None:
            table["head"] = ParamSpec((s.vocab_size, s.hidden), [Source(s.head_name)])
        for path, part in self._walk():
            for local, ps in part.param_specs().items():
                table[f"{path}.{local}"] = ps
        return table

    def streamed_weights(self) -> list[torch.Tensor]:
        """The weight matrices that steps of few rows stream (the head, and `Part.streamed_params` of
        every part), each tensor once."""
        seen: dict[int, torch.Tensor] = {id(self.head): self.head}  # (the head of a decode step has few rows too)
        for _, part in self._walk():
            for local in part.streamed_params():
                w = getattr(part, local)
                seen.setdefault(id(w), w)
        return list(seen.values())

    def scratch_bytes_per_token(self, esize: int) -> int:
        """Bytes of step scratch per token of a step, for an activation type of `esize` bytes:
        the 32-bit residual, and every named buffer once (all blocks share the buffers by name,
        so the widest of each kind counts: the sum over the kinds of part of their largest
        request)."""
        widest: dict[type, int] = {}
        for _, part in self._walk():
            n = part.scratch_elements_per_token()
            if n:
                widest[type(part)] = max(widest.get(type(part), 0), n)
        return 4 * self.spec.hidden + esize * sum(widest.values())

    def ignorable(self, name: str) -> bool:
        return any(name == pat or name.endswith(pat) for pat in self.spec.ignorable)

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        self.embed = params["embed"]
        self.head = params.get("head", self.embed)  # tied: one tensor serves both
        for path, part in self._walk():
            mine = {local: params[f"{path}.{local}"] for local in part.param_specs()}
            if mine:
                part.bind(mine)

    def parameters(self) -> dict[str, torch.Tensor]:
        out = {"embed": self.embed}
        if self.spec.head_name is not None:
            out["head"] = self.head
        for path, part in self._walk():
            for local in part.param_specs():
                out[f"{path}.{local}"] = getattr(part, local)
        return out

    # ---- the forward pass of one step ----------------------------------------------------
    def forward(self, ctx: StepContext, handles: list[Any], want_rows: torch.Tensor | None,
                num_want: int) -> torch.Tensor:
        """Run the tokens of `ctx` through the model; `handles[i]` is the cache handle of
        ``order[i]`` (or None).  Returns float32 logits ``[num_want, vocab]`` of the packed
        token rows `want_rows`."""
        s = self.spec
        n = ctx.num_tokens
        residual = ctx.scratch("residual", (n, s.hidden), torch.float32)
        K.embedding(self.embed, ctx.tokens, residual, deferred=ctx.deferred)
        if self.embed_position is not None:
            self.embed_position.on_embedding(residual, ctx)
        delta = None
        for i, (call, handle) in enumerate(zip(s.order, handles, strict=True)):
            # the norm that will receive this block's output, if it can be begun by the block's
            # last product (`Block.entry_norm`); the final norm is always a kernel of its own
            ctx.extra["next_norm"] = (self.blocks[s.order[i + 1].layer].entry_norm()
                                      if i + 1 < len(s.order) else None)
            delta = self.blocks[call.layer].forward(delta, residual, ctx, handle)
        logits = ctx.scratch("logits", (num_want, s.vocab_size), torch.float32)
        if num_want == 0:
            # still fold the last delta in?  Nothing reads the residual after the step.
            return logits
        assert want_rows is not None and want_rows.numel() == num_want
        normed = self.final_norm.forward(delta, residual, ctx, rows=want_rows)
        linear_f32_out(normed, self.head, logits)
        return logits
