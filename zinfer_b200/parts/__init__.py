from .base import (Block, BuildContext, FeedForward, KVCacheNeed, Mixer, Norm, Part, PositionEncoding, StateNeed,
                   TensorSpec, make_part, prefixed, register_part, take, unregister_part)
from .attention import GQAttention
from .block import PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .mlp import SwiGLUMLP
from .norm import RMSNorm
from .rope import NoPosition, RotaryPosition

for _kind, _cls in (("rmsnorm", RMSNorm), ("rope", RotaryPosition), ("no_position", NoPosition),
                    ("gqa_attention", GQAttention), ("swiglu_mlp", SwiGLUMLP), ("prenorm_block", PreNormBlock),
                    ("token_embedding", TokenEmbedding), ("lm_head", LMHead)):
    register_part(_kind, _cls, replace=True)

__all__ = [
    "Block", "BuildContext", "FeedForward", "GQAttention", "KVCacheNeed", "LMHead", "Mixer", "NoPosition", "Norm",
    "Part", "PositionEncoding", "PreNormBlock", "RMSNorm", "RotaryPosition", "StateNeed", "SwiGLUMLP", "TensorSpec",
    "TokenEmbedding", "make_part", "prefixed", "register_part", "take", "unregister_part",
]
