"""The pre-norm arrangement: h1 = h + mixer(norm(h)); h2 = h1 + ffn(norm(h1))
(src/model/layers/rmsnorm_gqa_swiglu_block.zig:86-88,161-163).

The residual stream ``h`` is 32-bit.  An update that has not yet been added is
carried as ``pending`` into the next norm, where the add is fused with the norm;
the block therefore returns its feed-forward's output instead of adding it."""
from __future__ import annotations

from .base import Block, make_part, prefixed, take


class PreNormBlock(Block):
    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.mixer = make_part(params["mixer"], ctx)
        self.feed_forward = make_part(params["feed_forward"], ctx)
        self.mixer_norm = make_part(params["mixer_norm"], ctx)
        self.ffn_norm = make_part(params["ffn_norm"], ctx)
        self._names = {
            "mixer": params.get("mixer_name", "mixer") + ".",
            "feed_forward": params.get("ffn_name", "feed_forward") + ".",
            "mixer_norm": params.get("mixer_norm_name", "mixer_norm") + ".",
            "ffn_norm": params.get("ffn_norm_name", "ffn_norm") + ".",
        }

    def _parts(self):
        return [(self._names[k], getattr(self, k)) for k in ("mixer_norm", "mixer", "ffn_norm", "feed_forward")]

    def tensor_specs(self):
        out = {}
        for prefix, part in self._parts():
            out.update(prefixed(prefix, part.tensor_specs()))
        return out

    def bind(self, tensors):
        for prefix, part in self._parts():
            part.bind(take(tensors, prefix))

    def forward(self, h, pending, step, cache):
        x = self.mixer_norm.forward(h, pending)
        a = self.mixer.forward(x, step, cache)
        x = self.ffn_norm.forward(h, a)
        return self.feed_forward.forward(x)
