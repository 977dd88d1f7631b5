"""Plain PyTorch references of the kernels, one per entry point of
``zinfer_b200.ops`` and with the same signature.  Written from the formulas (cited
in tests/plain_qwen3.py), with 32-bit arithmetic and simple loops; they share no
code with the kernels.  GPU tests compare each kernel with its reference; the
CPU tests of the engine's host logic put these in the kernels' place.
"""
from __future__ import annotations

import numpy as np
import torch


def embed_gather(table, ids, out=None):
    return table[ids.long()].to(torch.float32)


def add_rmsnorm(h, delta, weight, eps, out_dtype, rows=None, out=None):
    if rows is None:
        if delta is not None:
            h += delta.to(torch.float32)
        x = h
    else:   # picked rows (repeats allowed): h itself stays as it is
        x = h[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].to(torch.float32)
    ms = (x * x).mean(dim=-1, keepdim=True)
    inv = 1.0 / torch.sqrt(ms + torch.tensor(eps, dtype=torch.float32))
    return (x * weight * inv).to(out_dtype)


def residual_add(h, delta):
    h += delta.to(torch.float32)


SWIGLU_INTERLEAVE = 64


def interleave_gate_up(gate, up, block=64):
    I, K = gate.shape
    return torch.stack([gate.view(I // block, block, K), up.view(I // block, block, K)], dim=1).reshape(2 * I, K).contiguous()


def linear_swiglu(x, w_interleaved, out_dtype=None):
    return swiglu(linear(x, w_interleaved, out_dtype=torch.float32), interleave=64).to(out_dtype or x.dtype)


def swiglu(gate_up, out=None, out_dtype=None, interleave=0):
    I = gate_up.shape[1] // 2
    if interleave:
        blocks = gate_up.reshape(gate_up.shape[0], I // interleave, 2, interleave)
        gate_up = torch.cat([blocks[:, :, 0].reshape(-1, I), blocks[:, :, 1].reshape(-1, I)], dim=1)
    g, u = gate_up[:, :I].to(torch.float32), gate_up[:, I:].to(torch.float32)
    return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)


def rope_table(n_pos, head_dim, theta, device):
    half = head_dim // 2
    exponent = (np.arange(half, dtype=np.float32) * np.float32(2)) / np.float32(head_dim)
    p = np.power(np.float64(np.float32(theta)), exponent.astype(np.float64)).astype(np.float32)
    inv = (np.float32(1) / p).astype(np.float32)
    ang = (np.arange(n_pos, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    cos = torch.from_numpy(np.cos(ang.astype(np.float64)).astype(np.float32)).to(device)
    sin = torch.from_numpy(np.sin(ang.astype(np.float64)).astype(np.float32)).to(device)
    return cos, sin


def qk_norm_rope_store(qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps, cos, sin, positions,
                       k_cache, v_cache, slots, page_size, write_kv=True, out_dtype=None):
    T = qkv.shape[0]
    nq, nkv, d = num_heads, num_kv_heads, head_dim
    half = d // 2
    pos = positions.long()

    def norm_rope(x, w):  # x [T, heads, d] float32
        if w is not None:
            ms = (x * x).mean(dim=-1, keepdim=True)
            x = x * w * (1.0 / torch.sqrt(ms + torch.tensor(eps, dtype=torch.float32)))
        if cos is not None:
            c, s = cos[pos][:, None, :], sin[pos][:, None, :]
            a, b = x[..., :half], x[..., half:]
            x = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
        return x

    q = norm_rope(qkv[:, :nq * d].to(torch.float32).reshape(T, nq, d), q_weight)
    qkv[:, :nq * d] = q.reshape(T, nq * d).to(qkv.dtype)
    if not write_kv:
        return qkv
    k = norm_rope(qkv[:, nq * d:(nq + nkv) * d].to(torch.float32).reshape(T, nkv, d), k_weight).to(qkv.dtype)
    v = qkv[:, (nq + nkv) * d:(nq + 2 * nkv) * d].reshape(T, nkv, d)
    for t in range(T):
        slot = int(slots[t])
        k_cache[slot // page_size, :, slot % page_size, :] = k[t]
        v_cache[slot // page_size, :, slot % page_size, :] = v[t]
    return qkv


def linear(x, weight, out_dtype=None, out=None, allow_partials=False):
    y = x.to(torch.float32) @ weight.to(torch.float32).T
    return y.to(out_dtype or x.dtype)


def attention_tile_rows():
    return 16


def attention_prefill_tile_rows():
    return 128


def paged_attention(q, k_cache, v_cache, block_tables, cu_q, kv_lens, tile_seq, tile_q0, num_heads, num_kv_heads,
                    head_dim, page_size, window, scale, out=None):
    T = q.shape[0]
    nq, nkv, d = num_heads, num_kv_heads, head_dim
    g = nq // nkv
    o = torch.zeros((T, nq * d), dtype=torch.float32, device=q.device)
    n = kv_lens.shape[0]
    for s in range(n):
        a, b = int(cu_q[s]), int(cu_q[s + 1])
        kv_len = int(kv_lens[s])
        ctx = kv_len - (b - a)
        for t in range(a, b):
            pos = ctx + (t - a)
            lo = 0 if not window else max(0, pos - window + 1)
            js = torch.arange(lo, pos + 1, device=q.device)
            pages = block_tables[s, (js // page_size)].long()
            offs = js % page_size
            K = k_cache[pages, :, offs, :].to(torch.float32)   # [keys, nkv, d]
            V = v_cache[pages, :, offs, :].to(torch.float32)
            qt = q[t, :nq * d].to(torch.float32).reshape(nq, d)
            for h in range(nq):
                sc = (K[:, h // g, :] @ qt[h]) * scale
                p = torch.softmax(sc, dim=0)
                o[t, h * d:(h + 1) * d] = p @ V[:, h // g, :]
    return o.to(q.dtype)


def argmax(logits, out=None):
    return torch.argmax(logits, dim=-1).to(torch.int32)


def linear_argmax(x, weight):
    logits = linear(x, weight, out_dtype=torch.float32)
    return logits, argmax(logits)


def attention(q, k_cache, v_cache, block_tables, step, num_heads, num_kv_heads, head_dim, page_size, window, scale):
    return paged_attention(q, k_cache, v_cache, block_tables, step.cu_q, step.kv_lens, step.tile_seq, step.tile_q0,
                           num_heads, num_kv_heads, head_dim, page_size, window, scale)


def patch_tokens(ids, prev, dst, src):
    for i in range(dst.numel()):
        if int(dst[i]) >= 0:
            ids[int(dst[i])] = prev[int(src[i])]


def decode_fused_ok(dtype, num_heads, num_kv_heads, head_dim, step):
    return False


def count_tokens(counts_row, tokens):
    for t in tokens.tolist():
        counts_row[int(t)] += 1


def sample(logits, temperature, seeds, draw_index, top_k=None, top_p=None, min_p=None, repetition_penalty=None,
           presence_penalty=None, frequency_penalty=None, count_rows=None, counts=None, out=None):
    """The reference's chain per row (penalties, top-k, temperature, min-p, top-p, draw) with the
    host sampler of tests/plain_qwen3.py.  The uniform number of a draw comes from (seed, draw
    index) alone, as on the device, but by another generator: tokens are comparable with the
    kernel's only where the kept set has one member (greedy rows)."""
    import hashlib

    import plain_qwen3 as P

    R, V = logits.shape
    res = torch.empty((R,), dtype=torch.int32)
    get = lambda t, i, default: default if t is None else t[i].item()
    for i in range(R):
        row = logits[i].float().numpy()
        crow = int(get(count_rows, i, -1))
        if counts is not None and crow >= 0:
            hist = np.repeat(np.arange(V), counts[crow].numpy())
            row = P.adjusted_logits(row, hist.tolist(), get(repetition_penalty, i, 1.0), get(presence_penalty, i, 0.0),
                                    get(frequency_penalty, i, 0.0))
        T, k = float(temperature[i]), int(get(top_k, i, 0))
        if T <= 0.0 or k == 1:
            tok = int(np.argmax(row))
        else:
            p = P.kept_distribution(row, T, k, float(get(top_p, i, 1.0)), float(get(min_p, i, 0.0)))
            h = hashlib.sha256(f"{int(seeds[i])}:{int(draw_index[i])}".encode()).digest()
            u = int.from_bytes(h[:8], "little") / 2.0 ** 64
            tok = int(min(np.searchsorted(np.cumsum(p), u, side="right"), V - 1))
            if p[tok] == 0.0:
                tok = int(np.argmax(p))
        if counts is not None and crow >= 0:
            counts[crow, tok] += 1
        res[i] = tok
    return res
