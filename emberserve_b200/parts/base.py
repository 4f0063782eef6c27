"""Interfaces of the building parts of a decoder, and the registries they live in.

A model is an assembly of parts, chosen by its configuration layer by layer:

* a **mixer** moves information between the tokens of a request (attention here);
  it may own a cache entry: pages of keys and values, or a slot of fixed-size state;
* a **feed-forward** works on each token alone (dense SwiGLU here);
* a **norm** adds a sub-layer's output to the residual stream and normalises it;
* a **position encoding** tells a mixer (or the embedding) where a token stands;
* a **block** arranges a mixer, a feed-forward and their norms around the residual.

No part knows which model it is in: every size and constant is a field of the
part's *spec* (a dataclass with a ``kind``), and the checkpoint tensor names a part
reads are given to it by the architecture's builder.  ``register_part`` adds a new
kind without touching this package; ``build_part`` turns a spec into a part.

The reference has the same pieces as ``nn.Module`` classes tied to one config
(``emberserve/model/qwen2.py:30-164``); the packed ``[num_tokens, hidden]`` layout
and "the model never touches the cache" rule are kept (``emberserve/attn/base.py:4-15``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

# ---------------------------------------------------------------------------------------
# parameters and where they come from


@dataclass(frozen=True)
class Source:
    """One checkpoint tensor that fills (a row range of) a parameter."""

    name: str
    rows: tuple[int, int] | None = None  # destination rows [lo, hi) along dim 0; None = all


@dataclass
class ParamSpec:
    shape: tuple[int, ...]
    sources: list[Source]
    # "float": kept in the compute dtype, except that a tensor stored in 32 bits stays
    # 32-bit; "int": an integer table, held as int32.
    role: str = "float"
    # How the random-weights mode fills it: "normal" (matrices and embeddings),
    # "bias" (normal with the bias deviation), "ones" (norm gains), "zeros".
    init: str = "normal"


# ---------------------------------------------------------------------------------------
# what a mixer needs from the cache manager


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every token, in pages.  `window`: only the last `window`
    keys are ever read again (None = all), so older pages may be given back."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class FixedState:
    """State of fixed size per request (a recurrent or convolutional mixer)."""

    shape: tuple[int, ...]
    dtype: str = "float32"


CacheNeed = PagedKV | FixedState


@dataclass
class PagedKVHandle:
    """One cache entry of kind PagedKV as a mixer sees it during a step."""

    k: torch.Tensor  # [num_pages, num_kv_heads, page_size, head_dim]
    v: torch.Tensor
    block_tables: torch.Tensor  # [rows, max_pages] int32, page ids of this entry's group
    page_size: int
    window: int | None
    write: bool  # False: read what another layer call wrote in this step


@dataclass
class FixedStateHandle:
    state: torch.Tensor  # [num_slots, *shape]
    slots: torch.Tensor  # [rows] int32 slot of each row of the step
    write: bool


# ---------------------------------------------------------------------------------------
# the step as parts see it


@dataclass
class StepContext:
    """Everything about one step that a part may read.  Rows are requests; tokens are
    packed ``[num_tokens, ...]`` in row order (``emberserve/attn/base.py:4-15``)."""

    num_tokens: int
    num_rows: int
    dtype: torch.dtype  # activation dtype: float32 or bfloat16
    device: torch.device
    # device tensors, int32
    tokens: torch.Tensor  # [num_tokens] token ids
    positions: torch.Tensor  # [num_tokens] absolute position of each token
    row_of_token: torch.Tensor  # [num_tokens]
    cu_q: torch.Tensor  # [num_rows + 1] first packed token of each row
    starts: torch.Tensor  # [num_rows] tokens already cached before this step
    # host copies
    q_lens: list[int]
    start_list: list[int]
    max_q_len: int = 1
    max_ctx_len: int = 1
    # scratch buffers that live across steps: scratch(name, shape, dtype) -> tensor
    scratch: Callable[..., torch.Tensor] | None = None
    extra: dict[str, Any] = field(default_factory=dict)
    # int32 device tokens that earlier kernels of the stream have sampled; a token id -(k + 1)
    # in `tokens` stands for deferred[k] (the engine launches a step before it has read the
    # tokens of the step before)
    deferred: torch.Tensor | None = None

    @property
    def all_decode(self) -> bool:
        return self.max_q_len == 1


# ---------------------------------------------------------------------------------------
# a norm split between the products on either side of it


@dataclass
class NormRequest:
    """What a block asks of the LAST product of a sub-layer when the norm behind the sub-layer
    can be begun there (steps of few rows, where every kernel saved is microseconds): add the
    product into `residual` instead of returning it, and hand back `ScaledRows` for the norm
    with this `gain` and `eps`.  A sub-layer that does not know about this ignores it."""

    residual: torch.Tensor  # [num_tokens, width] float32, updated in place
    gain: torch.Tensor  # [width]
    eps: float


@dataclass
class ScaledRows:
    """Activations of a norm that is not finished yet: `x` holds residual * gain (activation
    dtype); row n still has to be multiplied by rsqrt(sumsq[:parts, n].sum() / width + eps).
    That factor is one number per row, so it commutes with a product x W^T: the product that
    reads `x` applies it to its result (`parts.linear`), and the norm costs no kernel of its own.
    `materialize()` finishes the norm the plain way for a reader that cannot."""

    x: torch.Tensor  # [num_tokens, width]
    sumsq: torch.Tensor  # [parts, 16] float32: shares of each row's sum of squares
    parts: int
    eps: float

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def is_cuda(self) -> bool:
        return self.x.is_cuda

    def materialize(self) -> torch.Tensor:
        n, width = self.x.shape
        total = self.sumsq[:self.parts, :n].sum(0)
        rstd = torch.rsqrt(total / width + self.eps)
        return (self.x.float() * rstd[:, None]).to(self.x.dtype)


# ---------------------------------------------------------------------------------------
# parts


class SharedParts:
    """Parts that several layers share (one rotary table for all of them): built once
    per distinct spec while a model is assembled."""

    def __init__(self) -> None:
        self._memo: dict[tuple[str, Any], Part] = {}

    def get(self, category: str, spec: Any) -> "Part":
        key = (category, spec)
        if key not in self._memo:
            self._memo[key] = build_part(category, spec, f"shared.{category}.{len(self._memo)}", self)
        return self._memo[key]

    def all(self) -> list["Part"]:
        return list(self._memo.values())


class Part:
    """Base of all parts.  `prefix` is the path of the part inside the model, used only
    to name its parameters in error messages and in the loader's table."""

    def __init__(self, spec: Any, prefix: str, shared: SharedParts | None = None) -> None:
        self.spec = spec
        self.prefix = prefix
        self.shared = shared if shared is not None else SharedParts()

    def param_specs(self) -> dict[str, ParamSpec]:
        """Local parameter name -> shape and checkpoint sources."""
        return {}

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        """Receive the loaded parameters (device tensors), keyed by local name."""
        for name, tensor in params.items():
            setattr(self, name, tensor)

    def children(self) -> dict[str, "Part"]:
        return {}

    def streamed_params(self) -> list[str]:
        """Local names of the weight matrices that `forward` hands to ``parts.linear`` in steps of few
        rows, where every weight is read once per step: the engine may keep a second, tiled copy of
        these for the weight-streaming kernels (``parts.linear.give_tiled_twin``).  Naming none is
        always right."""
        return []

    def scratch_elements_per_token(self) -> int:
        """Elements of the activation dtype that `forward` asks of ``ctx.scratch`` per token of a
        step, children not counted.  Only used to keep memory free for the steps when the
        cache is sized; a part that allocates by other means may leave it at 0 (small
        allocations are covered by a fixed workspace)."""
        return 0


class Norm(Part):
    def split_request(self, residual: torch.Tensor, ctx: StepContext) -> "NormRequest | None":
        """A `NormRequest` if, in this step, the norm can be begun by the product before it and
        finished by the product behind it (then `forward` will be handed the `ScaledRows` that
        came of it as `delta`, and passes them on); None (the default) if it is a kernel of its own."""
        return None

    def forward(self, delta: torch.Tensor | None, residual: torch.Tensor,
                ctx: StepContext, rows: torch.Tensor | None = None) -> torch.Tensor:
        """residual += delta (32-bit sum); return norm(residual) in the activation dtype.
        With `rows` (int32 packed token indices on the device; their count is ``rows.numel()``)
        only the rows ``residual[rows] + delta[rows]`` are normalised and returned, compactly,
        and the residual is left unchanged: that is how the decoder calls the final norm, on
        the rows whose logits are wanted."""
        raise NotImplementedError


class PositionEncoding(Part):
    """How positions reach the model.  A rotary kind returns its table; an absolute
    kind would add to the embedding in `on_embedding`."""

    def rotary(self, device: torch.device) -> tuple[torch.Tensor, int] | None:
        """(cos/sin table ``[max_pos, rotary_dim/2, 2]`` float32, rotary_dim) or None."""
        return None

    def on_embedding(self, hidden: torch.Tensor, ctx: StepContext) -> None:
        return None

    @property
    def max_positions(self) -> int | None:
        return None


class Mixer(Part):
    # True if `forward` takes `ScaledRows` for x (its first product finishes the norm) and looks
    # for a `NormRequest` in ctx.extra["norm_behind"] (its last product begins the next norm,
    # and `forward` then returns `ScaledRows`).  False: plain tensors in and out.
    splits_norms = False

    def cache_need(self) -> CacheNeed | None:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Any) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    splits_norms = False  # as for Mixer

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of a mixer, a feed-forward and their norms.  Works on the pair
    (delta, residual): `delta` is the previous sub-layer's output that has not been
    added to the 32-bit residual stream yet (None right after the embedding)."""

    def cache_need(self) -> CacheNeed | None:
        raise NotImplementedError

    def entry_norm(self) -> "Norm | None":
        """The norm that receives what the block is given, if the sub-layer behind that norm takes
        `ScaledRows`: the block BEFORE this one may then let its last product begin that norm
        (the decoder tells it through ctx.extra["next_norm"]).  None: hand me a plain delta."""
        return None

    def forward(self, delta: torch.Tensor | None, residual: torch.Tensor, ctx: StepContext,
                cache: Any) -> torch.Tensor:
        """Returns the new delta; `residual` is updated in place."""
        raise NotImplementedError


# ---------------------------------------------------------------------------------------
# registries: spec kind -> part class

_CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block")
_REGISTRY: dict[str, dict[str, type[Part]]] = {c: {} for c in _CATEGORIES}


def register_part(category: str, kind: str, cls: type[Part] | None = None):
    """Register `cls` as the part built for specs of `kind` in `category` (one of
    mixer, feed_forward, norm, position, block).  Usable as a decorator."""
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category {category!r}; one of {_CATEGORIES}")

    def deco(c: type[Part]) -> type[Part]:
        _REGISTRY[category][kind] = c
        return c

    return deco if cls is None else deco(cls)


def build_part(category: str, spec: Any, prefix: str, shared: SharedParts | None = None) -> Part:
    kind = getattr(spec, "kind", None)
    try:
        cls = _REGISTRY[category][kind]
    except KeyError:
        known = sorted(_REGISTRY.get(category, {}))
        raise KeyError(f"no {category} part of kind {kind!r} is registered "
                       f"(known: {known})") from None
    return cls(spec, prefix, shared)


def registered_kinds(category: str) -> list[str]:
    return sorted(_REGISTRY[category])
