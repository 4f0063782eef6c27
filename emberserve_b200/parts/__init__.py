"""Parts a decoder is assembled from.  Importing the package registers the built-in kinds."""

from emberserve_b200.parts import attention, block, mlp, norm, rope  # noqa: F401
from emberserve_b200.parts.base import (Block, FeedForward, FixedState, FixedStateHandle, Mixer,
                                        Norm, PagedKV, PagedKVHandle, ParamSpec, Part,
                                        PositionEncoding, Source, StepContext, build_part,
                                        register_part, registered_kinds)

__all__ = ["Block", "FeedForward", "FixedState", "FixedStateHandle", "Mixer", "Norm", "PagedKV",
           "PagedKVHandle", "ParamSpec", "Part", "PositionEncoding", "Source", "StepContext",
           "build_part", "register_part", "registered_kinds"]
