"""Rotary position encoding with half-split pairs (i, i + d/2).

angle[p, i] = p * theta^(-2i/d); o[i] = x[i] cos - x[i+d/2] sin;
o[i+d/2] = x[i] sin + x[i+d/2] cos  (``litelang/kernel/develop_rope/rope.py:225-234``,
table ``litelang/models/qwen2/layer/pre_layer.py:21-30``).  The reference fixes
theta at 1e6 and casts the tables to half precision; here theta and the table
length come from the configuration and the table stays float32.

The table is built on the host with float32 operations in a fixed order, so the
angles are the same numbers on both precisions' paths.
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import PositionEncoding, register_part


def rope_table(rot_dim: int, theta: float, max_positions: int) -> torch.Tensor:
    """float32 [max_positions, rot_dim]: cos of the angles, then sin of the angles."""
    freqs = 1.0 / theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim)
    angle = torch.arange(0, max_positions, dtype=torch.float32)[:, None] * freqs[None, :]
    return torch.cat((torch.cos(angle), torch.sin(angle)), dim=1).contiguous()


class RotaryHalfSplit(PositionEncoding):
    fuses_with_store = True

    def __init__(self, spec):
        super().__init__(spec)
        self.rot_dim = int(spec.params["rotary_dim"])
        self.theta = float(spec.params["theta"])
        self.max_positions = int(spec.params["max_positions"])
        if self.rot_dim % 2:
            raise ValueError(f"rotary_dim {self.rot_dim} must be even")
        self.table: Optional[torch.Tensor] = None

    _shared = {}

    def prepare(self, device) -> None:
        key = (self.rot_dim, self.theta, self.max_positions, str(device))
        tab = RotaryHalfSplit._shared.get(key)
        if tab is None:
            tab = rope_table(self.rot_dim, self.theta, self.max_positions).to(device)
            RotaryHalfSplit._shared[key] = tab
        self.table = tab

    def fused_table(self) -> torch.Tensor:
        return self.table

    def apply(self, qkv, positions, num_heads, num_kv_heads, head_dim, num_tokens) -> None:
        ops.bias_rope_store(qkv, None, positions, self.table, num_heads, num_kv_heads, head_dim,
                            None, None, None, 1, None, num_tokens)


register_part("position", "rope_half_split", RotaryHalfSplit)
