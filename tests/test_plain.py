"""The plain implementation itself (no GPU): the reference's hand-computed unit
vectors, and internal consistency (causality, head mapping, greedy)."""
import numpy as np
import torch

import plain_qwen3 as P
from conftest import TINY_A, TINY_B

F64 = torch.float64


def test_rmsnorm_vector_from_the_reference():
    # src/kernel/core/cpu.zig:193-204
    y = P.rmsnorm(torch.tensor([3.0, 4.0], dtype=F64), torch.tensor([1.0, 2.0], dtype=F64), 0.0)
    np.testing.assert_allclose(y.numpy(), [0.84852814, 2.2627418], rtol=1e-7)
    # per-head repeat: each head is normed on its own (cpu.zig:274-287)
    x = torch.tensor([[3.0, 4.0], [6.0, 8.0]], dtype=F64)
    y = P.rmsnorm(x, torch.tensor([1.0, 2.0], dtype=F64), 0.0)
    np.testing.assert_allclose(y.numpy(), [[0.84852814, 2.2627418]] * 2, rtol=1e-7)


def test_swiglu_vector_from_the_reference():
    # src/kernel/core/cpu.zig:233-245
    y = P.swiglu(torch.tensor([0.0, 1.0, -1.0], dtype=F64), torch.tensor([1.0, 2.0, 3.0], dtype=F64))
    np.testing.assert_allclose(y.numpy(), [0.0, 1.4621172, -0.8068243], rtol=1e-6)


def test_rope_identity_at_zero_and_pair_rotation_at_one():
    # src/kernel/attention/rope.zig:145-190
    cos, sin = P.rope_tables(2, 4, 10000.0)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]], dtype=F64)
    np.testing.assert_allclose(P.apply_rope(x, cos[:1], sin[:1]).numpy(), x.numpy())
    y = P.apply_rope(x, cos[1:2], sin[1:2]).numpy()[0, 0]
    a0, a1 = 1.0, 0.01
    want = [np.cos(a0) - 3 * np.sin(a0), 2 * np.cos(a1) - 4 * np.sin(a1),
            3 * np.cos(a0) + np.sin(a0), 4 * np.cos(a1) + 2 * np.sin(a1)]
    np.testing.assert_allclose(y, want, rtol=1e-6)


def test_attention_maps_query_heads_to_kv_heads_and_is_convex():
    # consecutive query heads share a kv head (src/model/layers/gqa_attention/spec.zig:19-25;
    # cases of src/kernel/attention/basic.zig:178-252)
    S, nq, nkv, d = 3, 4, 2, 2
    q = torch.zeros(S, nq, d, dtype=F64)
    k = torch.zeros(S, nkv, d, dtype=F64)
    v = torch.zeros(S, nkv, d, dtype=F64)
    v[:, 0, :] = 1.0
    v[:, 1, :] = 5.0
    o = P.attention(q, k, v)
    np.testing.assert_allclose(o[:, :2].numpy(), 1.0)
    np.testing.assert_allclose(o[:, 2:].numpy(), 5.0)
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(6, n, 8, generator=g, dtype=F64) for n in (4, 2, 2))
    o = P.attention(q, k, v)
    for t in range(6):   # a convex mix of the values seen so far
        assert (o[t, 0] <= v[:t + 1, 0].max(dim=0).values + 1e-12).all()
        assert (o[t, 0] >= v[:t + 1, 0].min(dim=0).values - 1e-12).all()
    np.testing.assert_allclose(o[0, 3].numpy(), v[0, 1].numpy())   # the first token sees only itself


def test_window_limits_the_keys():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(9, 1, 4, generator=g, dtype=F64) for _ in range(3))
    full, win = P.attention(q, k, v), P.attention(q, k, v, window=3)
    np.testing.assert_allclose(win[:3].numpy(), full[:3].numpy())
    np.testing.assert_allclose(win[8].numpy(), P.attention(q[6:], k[6:], v[6:])[2].numpy())


def _model(raw, seed):
    from zinfer_b200.config import Qwen3Config, qwen3_model_spec
    from zinfer_b200.engine.model import declared_tensors
    from zinfer_b200.weights import random_tensors

    cfg = Qwen3Config.from_dict(raw)
    w = {k: v.to(F64) for k, v in random_tensors(declared_tensors(qwen3_model_spec(cfg)), seed, torch.float32).items()}
    return raw, w


def test_forward_is_causal_and_tied_head_is_the_embedding():
    cfg, w = _model(TINY_A, 3)
    toks = [5, 200, 17, 3, 99, 42]
    full = P.forward(cfg, w, toks)
    assert full.shape == (6, 256)
    np.testing.assert_allclose(P.forward(cfg, w, toks[:4]).numpy(), full[:4].numpy(), rtol=1e-12, atol=1e-14)
    assert P.head_weight(cfg, w) is w["model.embed_tokens.weight"]
    cfg_b, w_b = _model(TINY_B, 4)
    assert P.head_weight(cfg_b, w_b) is w_b["lm_head.weight"]
    assert P.forward(cfg_b, w_b, [1, 2, 3]).shape == (3, 384)


def test_greedy_takes_the_first_maximum_and_feeds_it_back():
    cfg, w = _model(TINY_A, 5)
    out = P.greedy(cfg, w, [7, 8, 9], 4)
    toks = [7, 8, 9]
    for t in out:
        assert t == int(torch.argmax(P.forward(cfg, w, toks)[-1]))
        toks.append(t)


def test_sampler_reference_behaviours():
    # src/sampling/sampler.zig:203-268: top-k restricts the support, penalties flip the argmax, min-p drops the tail
    logits = np.array([1.0, 3.0, 2.0, 0.5, 2.9], dtype=np.float32)
    p = P.kept_distribution(logits, 1.0, top_k=2)
    assert set(np.nonzero(p)[0]) == {1, 4} and abs(p.sum() - 1) < 1e-12
    adj = P.adjusted_logits(logits, [1, 1], repetition_penalty=1.0, presence_penalty=0.5, frequency_penalty=0.3)
    assert np.argmax(adj) == 4 and abs(adj[1] - (3.0 - 0.5 - 0.6)) < 1e-6
    adj = P.adjusted_logits(np.array([-1.0, 2.0], dtype=np.float32), [0, 1], repetition_penalty=2.0)
    np.testing.assert_allclose(adj, [-2.0, 1.0])
    p = P.kept_distribution(logits, 1.0, min_p=0.5)
    assert set(np.nonzero(p)[0]) == {1, 4}
    p = P.kept_distribution(logits, 1.0, top_p=0.5)
    assert set(np.nonzero(p)[0]) == {1, 4}   # 3.0 alone has 0.37 of the mass; with 2.9 it passes one half
    p = P.kept_distribution(logits, 0.5, top_p=0.0)
    assert set(np.nonzero(p)[0]) == {1}
