"""Rotary position encoding, rotate-half ("NeoX") pairing: dimension i of a head pairs
with dimension i + rotary_dim/2.

``inv_freq[i] = 1 / theta^(2i / rotary_dim)`` and ``angle = pos * inv_freq[i]``, both in
float32, as ``emberserve/model/rope.py:68-82`` computes them; the table of (cos, sin) is
built once on the device by ``ems_rope_table`` and applied by the kernel that also writes
keys and values into the cache (``csrc/elementwise.cu``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import PositionEncoding, register_part


@dataclass(frozen=True)
class RotarySpec:
    rotary_dim: int  # how many leading dimensions of a head rotate (head_dim for Qwen2)
    theta: float
    max_positions: int
    kind: str = "rotary_neox"


def inv_frequencies(rotary_dim: int, theta: float) -> torch.Tensor:
    """float32 ``1 / theta^(2i/rotary_dim)``, i in [0, rotary_dim/2)."""
    exponent = torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim
    return 1.0 / (float(theta) ** exponent)


@register_part("position", "rotary_neox")
class RotaryNeox(PositionEncoding):
    def __init__(self, spec: RotarySpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.rotary_dim % 2 or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim must be a positive even number, got {spec.rotary_dim}")
        self._table: torch.Tensor | None = None

    @property
    def max_positions(self) -> int:
        return self.spec.max_positions

    def rotary(self, device: torch.device) -> tuple[torch.Tensor, int]:
        s: RotarySpec = self.spec
        if self._table is None or self._table.device != device:
            inv = inv_frequencies(s.rotary_dim, s.theta).to(device)
            self._table = K.rope_table(inv, s.max_positions)
        return self._table, s.rotary_dim
