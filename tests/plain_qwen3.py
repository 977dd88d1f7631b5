"""Plain, slow implementation of the Qwen3 dense decoder: the tests' oracle.

Whole sequences, no cache, one function per part, float64 arithmetic on the CPU.
It shares no code with ``zinfer_b200``: it reads config.json with ``json`` and the
weights through its own minimal safetensors reader below.

The reference project (NeoZedAtlas/Zinfer) is written in Zig and no Zig toolchain
exists in this environment, so its model code can be neither imported nor compiled
here: this file rests on the reference's formulas, cited function by function as
``path:line`` within that project, and on the small hand-computed vectors of its
unit tests (reproduced in tests/test_plain.py).
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

F64 = torch.float64


# --------------------------------------------------------------------------- files
def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


_NP = {"F32": np.float32, "F64": np.float64, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def read_safetensors(path: str) -> dict[str, torch.Tensor]:
    """8-byte little-endian header length, JSON header, raw data
    (src/format/safetensors.zig:188-234)."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + hlen].decode("utf-8"))
    data = raw[8 + hlen :]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        shape = info["shape"]
        if info["dtype"] == "BF16":
            # bf16 -> f32 is a 16-bit left shift (src/tensor/formats/bfloat16.zig:3-6)
            u16 = np.frombuffer(data[b:e], dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u16.view(np.float32).copy())
        else:
            t = torch.from_numpy(np.frombuffer(data[b:e], dtype=_NP[info["dtype"]]).copy())
        out[name] = t.reshape(shape)
    return out


def load_model(model_dir: str) -> tuple[dict, dict[str, torch.Tensor]]:
    cfg = read_config(model_dir)
    w = {k: v.to(F64) for k, v in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, w


# --------------------------------------------------------------------------- parts
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y_i = x_i * w_i / sqrt(mean(x^2) + eps) over the last axis
    (src/kernel/core/cpu.zig:112-128; eps is cast to f32 first,
    src/model/layers/decoder_only_stack.zig:28-29)."""
    eps32 = float(np.float32(eps))
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(ms + eps32)) * weight


def rope_tables(n_pos: int, head_dim: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [n_pos, d/2] in the reference's 32-bit recipe: exponent 2i/d, pow,
    reciprocal, position * inv_freq, cos and sin each rounded to f32
    (src/kernel/attention/rope.zig:25-35; theta cast to f32 at
    src/model/runtime/optimized_decoder/layer.zig:41)."""
    half = head_dim // 2
    i2 = np.arange(half, dtype=np.float32) * np.float32(2.0)
    exponent = (i2 / np.float32(head_dim)).astype(np.float32)
    powed = np.power(np.float32(theta).astype(np.float64), exponent.astype(np.float64)).astype(np.float32)
    inv_freq = (np.float32(1.0) / powed).astype(np.float32)
    pos = np.arange(n_pos, dtype=np.float32)[:, None]
    angle = (pos * inv_freq[None, :]).astype(np.float32)
    cos = np.cos(angle.astype(np.float64)).astype(np.float32)
    sin = np.sin(angle.astype(np.float64)).astype(np.float32)
    return torch.from_numpy(cos).to(F64), torch.from_numpy(sin).to(F64)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [S, heads, d]; pairs (i, i + d/2): x'_i = x_i cos - x_{i+h} sin,
    x'_{i+h} = x_{i+h} cos + x_i sin (src/kernel/attention/rope.zig:67-90)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None) -> torch.Tensor:
    """q [S, nq, d], k/v [S, nkv, d] -> [S, nq, d].  q head h reads kv head
    h // (nq/nkv) (src/model/layers/gqa_attention/spec.zig:19-25); the score is
    dot * 1/sqrt(d) (src/kernel/attention/basic.zig:49-64); softmax with the maximum
    subtracted (basic.zig:5-25); a token sees itself and everything before it
    (append precedes attention, src/model/runtime/optimized_decoder/layer.zig:130-142).
    ``window`` (not used by Qwen3; for the parts' tests) keeps keys j > i - window."""
    S, nq, d = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
    out = torch.empty_like(q)
    idx = torch.arange(S, device=q.device)
    mask = idx[None, :] <= idx[:, None]
    if window is not None:
        mask &= idx[None, :] > idx[:, None] - window
    for h in range(nq):
        kv = h // g
        s = (q[:, h, :] @ k[:, kv, :].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        e = torch.exp(s)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, kv, :]
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(g) * u with silu(x) = x / (1 + exp(-x)) (src/kernel/core/cpu.zig:130-147)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def attention_block(x, w, prefix, cfg, cos, sin):
    """q/k/v projections, per-head RMSNorm of q and k, RoPE, attention, o projection
    (src/model/runtime/optimized_decoder/layer.zig:110-142,188)."""
    S = x.shape[0]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = (x @ w[prefix + "self_attn.q_proj.weight"].T).reshape(S, nq, d)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].T).reshape(S, nkv, d)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].T).reshape(S, nkv, d)
    q = rmsnorm(q, w[prefix + "self_attn.q_norm.weight"], eps)
    k = rmsnorm(k, w[prefix + "self_attn.k_norm.weight"], eps)
    q = apply_rope(q, cos[:S], sin[:S])
    k = apply_rope(k, cos[:S], sin[:S])
    o = attention(q, k, v).reshape(S, nq * d)
    return o @ w[prefix + "self_attn.o_proj.weight"].T


def mlp_block(x, w, prefix):
    """gate and up projections, SwiGLU, down projection (layer.zig:193-197)."""
    g = x @ w[prefix + "mlp.gate_proj.weight"].T
    u = x @ w[prefix + "mlp.up_proj.weight"].T
    return swiglu(g, u) @ w[prefix + "mlp.down_proj.weight"].T


def decoder_layer(h, w, i, cfg, cos, sin):
    """h1 = h + attn(norm(h)); h2 = h1 + mlp(norm(h1)) (layer.zig:108,189-201)."""
    p = f"model.layers.{i}."
    eps = cfg["rms_norm_eps"]
    h = h + attention_block(rmsnorm(h, w[p + "input_layernorm.weight"], eps), w, p, cfg, cos, sin)
    h = h + mlp_block(rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps), w, p)
    return h


def head_weight(cfg, w):
    """lm_head.weight; with tie_word_embeddings the embedding table stands for it
    when the file has no separate head (the reference always looks lm_head.weight
    up by name, src/model/runtime/optimized_decoder/runtime.zig:50)."""
    if "lm_head.weight" in w and not cfg.get("tie_word_embeddings", False):
        return w["lm_head.weight"]
    if cfg.get("tie_word_embeddings", False):
        return w["model.embed_tokens.weight"]
    return w["lm_head.weight"]


def forward(cfg: dict, w: dict[str, torch.Tensor], tokens, rows=None) -> torch.Tensor:
    """Logits [S, V] for a whole sequence: embedding row, L layers, final norm, output
    head (src/model/runtime/optimized_decoder/runtime.zig:103-148).  Computed in the
    weights' dtype (float64 as :func:`load_model` gives them) and on their device; ``rows``
    restricts the output head to those positions (the layers always see the whole sequence)."""
    table = w["model.embed_tokens.weight"]
    tokens = torch.as_tensor(tokens, dtype=torch.long, device=table.device)
    S = tokens.shape[0]
    cos, sin = (t.to(device=table.device, dtype=table.dtype) for t in rope_tables(S, cfg["head_dim"], cfg["rope_theta"]))
    h = table[tokens]
    for i in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, i, cfg, cos, sin)
    h = rmsnorm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    if rows is not None:
        h = h[torch.as_tensor(list(rows), dtype=torch.long, device=h.device)]
    return h @ head_weight(cfg, w).T


def greedy(cfg, w, prompt, n_new: int) -> list[int]:
    """Greedy continuation; the first maximum wins (src/sampling/sampler.zig:93-105)."""
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(cfg, w, toks)[-1]
        nxt = int(torch.argmax(logits))  # torch.argmax returns the first maximum on CPU
        out.append(nxt)
        toks.append(nxt)
    return out


# ----------------------------------------------------------- sampler (host reference)
def adjusted_logits(logits: np.ndarray, history, repetition_penalty=1.0, presence_penalty=0.0,
                    frequency_penalty=0.0) -> np.ndarray:
    """Penalties in the reference's order (src/sampling/sampler.zig:186-201)."""
    out = logits.astype(np.float32).copy()
    counts: dict[int, int] = {}
    for t in history:
        if 0 <= t < len(out):
            counts[t] = counts.get(t, 0) + 1
    for t, c in counts.items():
        a = out[t]
        if repetition_penalty > 0.0 and repetition_penalty != 1.0:
            a = a * np.float32(repetition_penalty) if a < 0 else a / np.float32(repetition_penalty)
        a = a - np.float32(presence_penalty)
        a = a - np.float32(c) * np.float32(frequency_penalty)
        out[t] = a
    return out


def kept_distribution(logits: np.ndarray, temperature: float, top_k: int = 0, top_p: float = 1.0,
                      min_p: float = 0.0) -> np.ndarray:
    """Probability of each token after top-k, temperature, min-p, top-p in the
    reference's order (src/sampling/sampler.zig:35-90).  Ties at the top-k edge
    are broken toward the lower token id."""
    V = len(logits)
    k = V if top_k == 0 else min(top_k, V)
    order = np.lexsort((np.arange(V), -logits.astype(np.float64)))[:k]
    z = logits[order].astype(np.float32) / np.float32(temperature)
    e = np.exp((z - z.max()).astype(np.float32)).astype(np.float64)
    keep = k
    mp = min(max(min_p, 0.0), 1.0)
    if mp > 0.0:
        thr = np.float32(e[0]) * np.float32(mp)
        keep = 0
        while keep < k and e[keep] >= thr:
            keep += 1
        keep = max(keep, 1)
    s = e[:keep].sum()
    tp = min(max(top_p, 0.0), 1.0)
    if tp < 1.0:
        cum = 0.0
        n = 0
        while n < keep:
            cum += e[n] / s
            n += 1
            if cum >= tp:
                break
        keep = min(max(n, 1), keep)
    p = np.zeros(V, dtype=np.float64)
    p[order[:keep]] = e[:keep] / e[:keep].sum()
    return p
