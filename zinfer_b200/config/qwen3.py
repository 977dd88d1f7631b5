"""Typed configuration of Qwen3 dense, read from the keys of its config.json.

Keys and their meaning follow the reference's ``Config`` struct
(src/model/families/qwen3/config.zig:3-23): every size and constant the model uses
comes from here; none is written in code.  Unknown keys are ignored as the
reference does (config.zig:40-42), except those that would change the arithmetic
if honoured (rope scaling, sliding windows, biases, another activation): these are
refused with a clear error rather than silently dropped.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field

from .spec import LayerSpec, ModelSpec, PartSpec, default_schedule


class ConfigError(ValueError):
    pass


_REQUIRED = (
    "hidden_size",
    "intermediate_size",
    "max_position_embeddings",
    "num_attention_heads",
    "num_hidden_layers",
    "num_key_value_heads",
    "rms_norm_eps",
    "rope_theta",
    "vocab_size",
)


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    model_type: str = "qwen3"
    architectures: tuple[str, ...] = ("Qwen3ForCausalLM",)
    eos_token_id: tuple[int, ...] = field(default_factory=tuple)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {', '.join(missing)}")
        for key, bad in (
            ("rope_scaling", lambda v: v is not None),
            ("use_sliding_window", lambda v: bool(v)),
            ("attention_bias", lambda v: bool(v)),
            ("hidden_act", lambda v: v != "silu"),
        ):
            if key in d and bad(d[key]):
                raise ConfigError(f"config.json: {key}={d[key]!r} is not supported by the Qwen3 dense family")
        nq = int(d["num_attention_heads"])
        head_dim = d.get("head_dim")
        if head_dim is None:  # older configs omit it; the width then fixes it
            if int(d["hidden_size"]) % nq:
                raise ConfigError("head_dim is absent and hidden_size is not a multiple of num_attention_heads")
            head_dim = int(d["hidden_size"]) // nq
        eos = d.get("eos_token_id", ())
        if isinstance(eos, int):
            eos = (eos,)
        cfg = cls(
            vocab_size=int(d["vocab_size"]),
            hidden_size=int(d["hidden_size"]),
            intermediate_size=int(d["intermediate_size"]),
            num_hidden_layers=int(d["num_hidden_layers"]),
            num_attention_heads=nq,
            num_key_value_heads=int(d["num_key_value_heads"]),
            head_dim=int(head_dim),
            max_position_embeddings=int(d["max_position_embeddings"]),
            rms_norm_eps=float(d["rms_norm_eps"]),
            rope_theta=float(d["rope_theta"]),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            model_type=str(d.get("model_type", "qwen3")),
            architectures=tuple(d.get("architectures", ("Qwen3ForCausalLM",))),
            eos_token_id=tuple(int(t) for t in (eos or ())),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "Qwen3Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        if os.path.getsize(path) > 1024 * 1024:  # the reference's limit, config.zig:39
            raise ConfigError(f"{path}: larger than 1 MiB")
        with open(path) as f:
            try:
                d = json.load(f)
            except json.JSONDecodeError as e:
                raise ConfigError(f"{path}: invalid JSON: {e}") from None
        if not isinstance(d, dict):
            raise ConfigError(f"{path}: top level is not an object")
        return cls.from_dict(d)

    def validate(self) -> None:
        """Checks of src/model/layers/rmsnorm_gqa_swiglu_block.zig:34-40 and
        src/kernel/attention/rope.zig:16."""
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, k) <= 0:
                raise ConfigError(f"{k} must be positive, got {getattr(self, k)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) is not a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim must be even for rotary pairs, got {self.head_dim}")
        if not self.rms_norm_eps >= 0.0:
            raise ConfigError(f"rms_norm_eps must be >= 0, got {self.rms_norm_eps}")
        if not self.rope_theta > 0.0:
            raise ConfigError(f"rope_theta must be > 0, got {self.rope_theta}")

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        else:
            d.pop("eos_token_id")
        return d


# ---------------------------------------------------------------------- the family
# End-of-sequence ids of the published Qwen3 vocabularies
# (src/model/families/qwen3/generation_policy.zig:3).  They apply only when the
# configuration names none itself and its vocabulary is large enough to hold them.
_QWEN3_EOS = (151645, 151643)


def qwen3_model_spec(cfg: Qwen3Config) -> ModelSpec:
    """Qwen3 dense as parts: every layer is a pre-norm block of grouped-query
    attention (per-head RMSNorm on q and k, then rotary positions) and a SwiGLU
    feed-forward (src/model/families/qwen3/layout.zig:3-6,
    src/model/runtime/optimized_decoder/layer.zig:98-202)."""
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    position = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                 "max_positions": cfg.max_position_embeddings})
    mixer = PartSpec("gqa_attention", {
        "hidden_size": cfg.hidden_size,
        "num_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim,
        "qk_norm_eps": cfg.rms_norm_eps,     # Qwen3 norms q and k per head with the model's eps
        "window": None,                      # every key is visible
        "position": position,
    })
    ffn = PartSpec("swiglu_mlp", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
    block = PartSpec("prenorm_block", {
        "mixer": mixer, "mixer_norm": norm, "mixer_norm_name": "input_layernorm",
        "feed_forward": ffn, "ffn_norm": norm, "ffn_norm_name": "post_attention_layernorm",
        "mixer_name": "self_attn", "ffn_name": "mlp",
    })
    layers = tuple(LayerSpec(block=block, prefix=f"model.layers.{i}.") for i in range(cfg.num_hidden_layers))
    eos = cfg.eos_token_id or tuple(t for t in _QWEN3_EOS if t < cfg.vocab_size)
    return ModelSpec(
        architecture="Qwen3ForCausalLM",
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                               "name": "model.embed_tokens"}),
        layers=layers,
        schedule=default_schedule(len(layers)),
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps, "name": "model.norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                  "name": "lm_head", "tied_to": "model.embed_tokens" if cfg.tie_word_embeddings else None}),
        eos_token_ids=eos,
    )
