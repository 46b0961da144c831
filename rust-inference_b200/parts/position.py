"""Position encodings.

``rope``: rotate-half rotary encoding.  inv_freq[i] = 1 / theta^(2i/rotary_dim)
with theta and the power in float32, angle = float32(position) * inv_freq[i] as
a float32 product (thanhauco/rust-inference src/ops/rope.rs:19-47; theta is read
as float32, src/models/config.rs:33-34).  The table holds cos and sin of that
float32 angle, evaluated in float64 and rounded once, times ``scaling``.
The attention kernel applies the table itself (``fused_table``).  Parts with
the same rotary size, base, scaling and device share one table (a model's layers
usually do), so it is held once, not once per layer.

``none``: nothing.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding
from .registry import register_position


_shared_tables = {}        # (device, rot, float32 theta, scaling) -> table [positions, rot/2, 2]


@register_position("rope")
class Rope(PositionEncoding):
    graph_safe = True
    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.rot % 2 or spec.rot > spec.head_dim or spec.rot <= 0:
            raise ValueError(f"rotary_dim {spec.rot} must be even and within head_dim {spec.head_dim}")
        self._table = None

    def inv_freq(self) -> np.ndarray:
        rot = self.spec.rot
        theta = np.float32(self.spec.theta)
        exps = np.arange(0, rot, 2, dtype=np.float32) / np.float32(rot)
        return (np.float32(1.0) / np.power(theta, exps, dtype=np.float32)).astype(np.float32)

    def prepare(self, max_positions: int) -> None:
        if self._table is not None and self._table.shape[0] >= max_positions:
            return
        key = (str(self.env.device), int(self.spec.rot), float(np.float32(self.spec.theta)), float(self.spec.scaling))
        shared = _shared_tables.get(key)
        if shared is not None and shared.shape[0] >= max_positions:
            self._table = shared
            return
        pos = np.arange(max_positions, dtype=np.float32)
        ang = (pos[:, None] * self.inv_freq()[None, :]).astype(np.float32).astype(np.float64)
        scale = float(self.spec.scaling)
        table = np.stack([np.cos(ang) * scale, np.sin(ang) * scale], axis=-1).astype(np.float32)
        self._table = _shared_tables[key] = torch.from_numpy(table).to(self.env.device).contiguous()

    def fused_table(self):
        return self._table


@register_position("none")
class NoPosition(PositionEncoding):
    graph_safe = True
