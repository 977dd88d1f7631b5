"""Grouped-query attention over the paged cache.

q = Wq x, k = Wk x, v = Wv x (one fused product); optional RMSNorm of every q and k
head with a shared [d] weight, before the position encoding; k (normed, rotated)
and v (raw) go into the request's pages; every query reads the keys at or before
its position (within ``window`` if one is set); softmax of dot * 1/sqrt(d) in
32-bit; output projection.  Query head h reads kv head h // (num_heads/num_kv_heads).
(src/model/runtime/optimized_decoder/layer.zig:110-142,188;
src/model/layers/gqa_attention/spec.zig:3-26; src/kernel/attention/basic.zig:27-76.)
The head size is independent of the model width.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .base import KVCacheNeed, Mixer, TensorSpec, make_part


class GQAttention(Mixer):
    graph_safe = True   # forward() only launches kernels on device arrays: a decode step can be captured

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.nq = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        if self.nkv <= 0 or self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads do not divide into {self.nkv} kv heads")
        eps = params.get("qk_norm_eps")
        self.qk_norm_eps = None if eps is None else float(eps)
        self.window = params.get("window")
        self.position = make_part(params["position"], ctx) if params.get("position") is not None else None
        # 1/sqrt(d) as a 32-bit value, applied to the score after the dot (basic.zig:50)
        self.scale = float(np.float32(1.0) / np.sqrt(np.float32(self.d)))
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    # ------------------------------------------------------------------ weights
    def tensor_specs(self):
        q, kv = self.nq * self.d, self.nkv * self.d
        specs = {
            "q_proj.weight": TensorSpec((q, self.hidden)),
            "k_proj.weight": TensorSpec((kv, self.hidden)),
            "v_proj.weight": TensorSpec((kv, self.hidden)),
            "o_proj.weight": TensorSpec((self.hidden, q)),
        }
        if self.qk_norm_eps is not None:
            specs["q_norm.weight"] = TensorSpec((self.d,), init="norm")
            specs["k_norm.weight"] = TensorSpec((self.d,), init="norm")
        return specs

    def bind(self, tensors):
        parts = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        if len({p.dtype for p in parts}) > 1:
            parts = [p.to(torch.float32) for p in parts]
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.qk_norm_eps is not None:
            self.q_norm = tensors["q_norm.weight"].to(torch.float32).contiguous()
            self.k_norm = tensors["k_norm.weight"].to(torch.float32).contiguous()

    # -------------------------------------------------------------------- cache
    def cache_need(self):
        return KVCacheNeed(num_kv_heads=self.nkv, head_dim=self.d, window=self.window)

    def max_positions(self):
        return None if self.position is None else getattr(self.position, "n_positions", None)

    # ------------------------------------------------------------------ forward
    def forward(self, x, step, cache):
        q_width = self.nq * self.d
        w = self.w_qkv if cache.writes else self.w_qkv[:q_width]  # a reader of another's cache needs q only
        qkv = ops.linear(x, w, out_dtype=self.ctx.dtype, allow_partials=True)
        group = step.kv_groups[cache.group]
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        if cache.writes and ops.decode_fused_ok(self.ctx.dtype, self.nq, self.nkv, self.d, step):
            # every request brings one token: norm, rotation, cache write and attention are one kernel
            o = ops.attention_decode_fused(
                qkv, self.nq, self.nkv, self.d, self.q_norm, self.k_norm,
                self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, cos, sin, cache.k, cache.v,
                group.slot_mapping, group.block_tables, step, cache.page_size, self.window, self.scale)
            return ops.linear(o, self.w_o, out_dtype=self.ctx.dtype, allow_partials=True)
        q = ops.qk_norm_rope_store(
            qkv, self.nq, self.nkv, self.d, self.q_norm, self.k_norm,
            self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, cos, sin, step.positions,
            cache.k, cache.v, group.slot_mapping, cache.page_size, write_kv=cache.writes, out_dtype=self.ctx.dtype)
        o = ops.attention(q, cache.k, cache.v, group.block_tables, step, self.nq, self.nkv, self.d,
                          cache.page_size, self.window, self.scale)
        return ops.linear(o, self.w_o, out_dtype=self.ctx.dtype, allow_partials=True)
