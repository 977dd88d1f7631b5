"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x))
(src/model/runtime/optimized_decoder/layer.zig:193-197, src/kernel/core/cpu.zig:130-147).
gate and up are stored as one matrix [2I, H] so one product feeds both."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec


class SwiGLUMLP(FeedForward):
    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.w_gate_up = None
        self.w_down = None

    def tensor_specs(self):
        return {
            "gate_proj.weight": TensorSpec((self.inter, self.hidden)),
            "up_proj.weight": TensorSpec((self.inter, self.hidden)),
            "down_proj.weight": TensorSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        # rows interleaved in blocks of 64 (gate block, up block) when the width allows it: the
        # tensor-core product can then apply the SwiGLU in its epilogue
        self.interleaved = self.inter % ops.SWIGLU_INTERLEAVE == 0
        self.w_gate_up = ops.interleave_gate_up(g, u) if self.interleaved else torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, x):
        if self.interleaved:
            act = ops.linear_swiglu(x, self.w_gate_up, out_dtype=self.ctx.dtype)
        else:
            gu = ops.linear(x, self.w_gate_up, out_dtype=self.ctx.dtype, allow_partials=True)
            act = ops.swiglu(gu, out_dtype=self.ctx.dtype)
        # the product may come back as split-K partial sums; the next norm adds them with the residual
        return ops.linear(act, self.w_down, out_dtype=self.ctx.dtype, allow_partials=True)
