"""Token embedding and output head
(src/model/runtime/optimized_decoder/runtime.zig:109-115,139-146)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorSpec


class TokenEmbedding(Part):
    """h0 = table[token]; no scaling.  Gives the 32-bit residual stream."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.name = params.get("name", "embed_tokens")
        self.weight = None

    def tensor_specs(self):
        return {self.name + ".weight": TensorSpec((self.vocab, self.hidden))}

    def bind(self, tensors):
        self.weight = tensors[self.name + ".weight"].contiguous()

    def forward(self, token_ids):
        return ops.embed_gather(self.weight, token_ids)


class LMHead(Part):
    """logits = W x in 32-bit.  ``tied_to`` names the embedding whose table stands
    for W; a separate ``<name>.weight`` in the file is then optional and unused."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.name = params.get("name", "lm_head")
        self.tied_to = params.get("tied_to")
        self.weight = None

    def tensor_specs(self):
        return {self.name + ".weight": TensorSpec((self.vocab, self.hidden), optional=self.tied_to is not None)}

    def bind(self, tensors):
        if self.tied_to is None:
            self.weight = tensors[self.name + ".weight"].contiguous()

    def tie(self, table: torch.Tensor):
        self.weight = table

    def forward(self, x):
        return ops.linear(x, self.weight, out_dtype=torch.float32)

    def forward_argmax(self, x):
        """The logits and each row's first maximum, found in the product's own epilogue where the
        tensor-core kernel takes the shape."""
        return ops.linear_argmax(x, self.weight)
