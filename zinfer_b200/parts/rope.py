"""Rotary position encoding, rotate-half pairing (i, i + d/2) over the whole head
(src/kernel/attention/rope.zig:67-90).  The part owns the cos/sin table, built on
the device by the reference's 32-bit recipe (rope.zig:25-35); equal parts share
one table."""
from __future__ import annotations

from .. import ops
from .base import PositionEncoding


class RotaryPosition(PositionEncoding):
    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.head_dim = int(params["head_dim"])
        self.theta = float(params["theta"])
        if self.head_dim % 2:
            raise ValueError(f"rotary positions need an even head_dim, got {self.head_dim}")
        # a request is never longer than the engine's limit nor than the model's own
        self.n_positions = min(int(params["max_positions"]), ctx.max_positions)
        self._key = ("rope", self.head_dim, self.theta, self.n_positions)

    def tables(self):
        """cos and sin [positions, d/2], built on the device at first use."""
        shared = self.ctx.shared
        if self._key not in shared:
            shared[self._key] = ops.rope_table(self.n_positions, self.head_dim, self.theta, self.ctx.device)
        return shared[self._key]


class NoPosition(PositionEncoding):
    """A mixer without position encoding."""

    n_positions = None

    def tables(self):
        return None, None
