"""Each part alone, built from its PartSpec at sizes other than the tiny models',
against the plain functions of tests/plain_qwen3.py."""
import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def _ctx(dtype):
    from zinfer_b200.parts import BuildContext
    return BuildContext(device=torch.device(DEV), dtype=dtype, max_positions=512)


def _bind(part, dtype, seed=0):
    from zinfer_b200.weights import random_tensors
    t = random_tensors(part.tensor_specs(), seed, dtype, DEV)
    part.bind(t)
    return {k: v.detach().cpu().to(F64) for k, v in t.items()}


def _tol(dtype):
    return dict(rtol=3e-5, atol=3e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part_adds_then_norms(dtype):
    from zinfer_b200.config import PartSpec
    from zinfer_b200.parts import make_part

    part = make_part(PartSpec("rmsnorm", {"size": 136, "eps": 1e-5}), _ctx(dtype))
    w = _bind(part, dtype)
    h = torch.randn(5, 136, device=DEV)
    delta = torch.randn(5, 136, device=DEV).to(dtype)
    want_h = h.cpu().to(F64) + delta.cpu().to(F64)
    got = part.forward(h, delta)
    torch.testing.assert_close(h.cpu().to(F64), want_h, rtol=1e-6, atol=1e-6)      # the residual is updated in place, in 32-bit
    torch.testing.assert_close(got.cpu().to(F64), P.rmsnorm(want_h, w["weight"], 1e-5), **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mlp_part(dtype):
    from zinfer_b200.config import PartSpec
    from zinfer_b200.parts import make_part

    part = make_part(PartSpec("swiglu_mlp", {"hidden_size": 72, "intermediate_size": 200}), _ctx(dtype))
    w = _bind(part, dtype, seed=1)
    x = torch.randn(9, 72, device=DEV).to(dtype)
    got = part.forward(x)
    if not isinstance(got, torch.Tensor):
        got = got.sum(dtype)
    xd = x.cpu().to(F64)
    want = P.swiglu(xd @ w["gate_proj.weight"].T, xd @ w["up_proj.weight"].T) @ w["down_proj.weight"].T
    torch.testing.assert_close(got.cpu().to(F64), want, rtol=_tol(dtype)["rtol"], atol=_tol(dtype)["atol"] * 0.05)


def test_rotary_part_shares_equal_tables():
    from zinfer_b200.config import PartSpec
    from zinfer_b200.parts import make_part

    ctx = _ctx(torch.float32)
    a = make_part(PartSpec("rope", {"head_dim": 48, "theta": 5e4, "max_positions": 300}), ctx)
    b = make_part(PartSpec("rope", {"head_dim": 48, "theta": 5e4, "max_positions": 300}), ctx)
    c = make_part(PartSpec("rope", {"head_dim": 48, "theta": 1e4, "max_positions": 300}), ctx)
    assert a.tables()[0] is b.tables()[0] and a.tables()[0] is not c.tables()[0]
    cos, sin = P.rope_tables(300, 48, 5e4)
    np.testing.assert_allclose(a.tables()[0].cpu().numpy(), cos.numpy().astype(np.float32), atol=4e-5)
    np.testing.assert_allclose(a.tables()[1].cpu().numpy(), sin.numpy().astype(np.float32), atol=4e-5)


def _attention_case(dtype, window, qk_norm, lens):
    from zinfer_b200.cache import CacheManager, CacheStorage
    from zinfer_b200.config import PartSpec
    from zinfer_b200.engine import StepEntry, build_step
    from zinfer_b200.parts import make_part
    from zinfer_b200 import ops

    H, nq, nkv, d, page = 88, 6, 2, 64, 8
    rope = PartSpec("rope", {"head_dim": d, "theta": 2e4, "max_positions": 400})
    spec = PartSpec("gqa_attention", {"hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d,
                                      "qk_norm_eps": 1e-6 if qk_norm else None, "window": window, "position": rope})
    part = make_part(spec, _ctx(dtype))
    w = _bind(part, dtype, seed=3)
    mgr = CacheManager({"c": part.cache_need()}, [], page, 64, 4)
    storage = CacheStorage(mgr, {}, dtype, DEV)
    view = storage.kv_view("c", True)
    g = torch.Generator().manual_seed(1)
    xs = {i: torch.randn(n, H, generator=g).to(dtype) for i, n in enumerate(lens)}
    outs = {i: [] for i in xs}
    # feed every request in two portions, the second beside the first of the next one
    cuts = {i: max(1, n // 3) for i, n in enumerate(lens)}
    steps = [[(i, 0, cuts[i]) for i in xs], [(i, cuts[i], lens[i]) for i in xs]]
    for st in steps:
        entries = []
        for i, a, b in st:
            if not mgr.has_request(i):
                mgr.add_request(i)
            mgr.reserve(i, b - a)
            entries.append(StepEntry(i, [0] * (b - a), []))
        ctx = build_step(mgr, entries, DEV, ops.attention_tile_rows(), pf_tile_rows=ops.attention_prefill_tile_rows())
        x = torch.cat([xs[i][a:b] for i, a, b in st]).to(DEV)
        y = part.forward(x, ctx, view)
        if not isinstance(y, torch.Tensor):
            y = y.sum(dtype)
        o = 0
        for i, a, b in st:
            outs[i].append(y[o:o + b - a].cpu())
            o += b - a
            mgr.commit(i, b - a)
    for i, n in enumerate(lens):
        xd = xs[i].to(F64)
        q = (xd @ w["q_proj.weight"].T).reshape(n, nq, d)
        k = (xd @ w["k_proj.weight"].T).reshape(n, nkv, d)
        v = (xd @ w["v_proj.weight"].T).reshape(n, nkv, d)
        if qk_norm:
            q, k = P.rmsnorm(q, w["q_norm.weight"], 1e-6), P.rmsnorm(k, w["k_norm.weight"], 1e-6)
        cos, sin = P.rope_tables(n, d, 2e4)
        q, k = P.apply_rope(q, cos, sin), P.apply_rope(k, cos, sin)
        want = P.attention(q, k, v, window=window).reshape(n, nq * d) @ w["o_proj.weight"].T
        got = torch.cat(outs[i]).to(F64)
        t = _tol(dtype)
        torch.testing.assert_close(got, want, rtol=t["rtol"], atol=t["atol"] * 0.1)
    mgr.check()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,qk_norm", [(None, True), (11, False)])
def test_attention_part_over_pages(dtype, window, qk_norm):
    _attention_case(dtype, window, qk_norm, lens=[37, 5, 70])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_part_carries_the_pending_update(dtype):
    """h1 = h + mixer(norm(h)); the block returns the feed-forward's output for the next norm to add."""
    from zinfer_b200.config import PartSpec
    from zinfer_b200.parts import Mixer, make_part, register_part, unregister_part

    class Doubler(Mixer):          # a mixer without weights or cache: y = 2x
        def forward(self, x, step, cache):
            return (x.float() * 2).to(x.dtype)

    register_part("toy_doubler", Doubler)
    try:
        norm = PartSpec("rmsnorm", {"size": 64, "eps": 1e-6})
        spec = PartSpec("prenorm_block", {"mixer": PartSpec("toy_doubler", {}), "mixer_norm": norm, "ffn_norm": norm,
                                          "feed_forward": PartSpec("swiglu_mlp", {"hidden_size": 64, "intermediate_size": 96})})
        block = make_part(spec, _ctx(dtype))
        assert set(block.tensor_specs()) == {"mixer_norm.weight", "ffn_norm.weight", "feed_forward.gate_proj.weight",
                                             "feed_forward.up_proj.weight", "feed_forward.down_proj.weight"}
        w = _bind(block, dtype, seed=4)
        h = torch.randn(6, 64, device=DEV)
        pending = torch.randn(6, 64, device=DEV).to(dtype)
        h0 = h.cpu().to(F64) + pending.cpu().to(F64)
        out = block.forward(h, pending, None, None)
        if not isinstance(out, torch.Tensor):
            out = out.sum(dtype)
        h1 = h0 + 2 * P.rmsnorm(h0, w["mixer_norm.weight"], 1e-6)
        x = P.rmsnorm(h1, w["ffn_norm.weight"], 1e-6)
        want = P.swiglu(x @ w["feed_forward.gate_proj.weight"].T, x @ w["feed_forward.up_proj.weight"].T) \
            @ w["feed_forward.down_proj.weight"].T
        t = _tol(dtype)
        torch.testing.assert_close(h.cpu().to(F64), h1, rtol=t["rtol"], atol=t["atol"])
        torch.testing.assert_close(out.cpu().to(F64), want, rtol=t["rtol"], atol=t["atol"] * 0.05)
    finally:
        unregister_part("toy_doubler")
