"""Each kernel alone against its plain PyTorch reference (tests/kernel_refs.py), in
float32 and bfloat16, at sizes other than the engine's tiny models: widths and
vocabularies that are no powers of two, head sizes in steps of 16, odd head counts."""
import numpy as np
import pytest
import torch

import kernel_refs as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from zinfer_b200 import ops as o
    return o


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-3)


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def test_library_is_loaded_from_the_tree():
    import os
    path = ops().library_file()
    assert os.path.exists(path) and path.endswith(".so")
    ops().lib()
    with open("/proc/self/maps") as f:
        assert "libzinfer_b200.so" in f.read(), "the kernel library is not mapped into the process"


def test_no_cpu_path():
    o = ops()
    with pytest.raises(o.KernelError):
        o.swiglu(torch.zeros(2, 4))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,H,T", [(301, 72, 9), (1000, 4096, 3), (17, 16, 33)])
def test_embed_gather(dtype, V, H, T):
    table = rnd(V, H, dtype=dtype)
    ids = torch.randint(0, V, (T,), dtype=torch.int32, device=DEV)
    got = ops().embed_gather(table, ids)
    assert got.dtype == torch.float32
    torch.testing.assert_close(got, ref.embed_gather(table, ids), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,eps", [(5, 72, 1e-6), (3, 4096, 1e-5), (130, 200, 3e-6), (2, 5120, 1e-6)])
def test_add_rmsnorm(dtype, T, H, eps):
    h = rnd(T, H, scale=3.0)
    delta = rnd(T, H, dtype=dtype, seed=1)
    w = 1 + 0.1 * rnd(H, seed=2)
    for d in (None, delta):
        h_ref, h_got = h.clone(), h.clone()
        want = ref.add_rmsnorm(h_ref, d, w, eps, dtype)
        got = ops().add_rmsnorm(h_got, d, w, eps, dtype)
        torch.testing.assert_close(h_got, h_ref, rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=DEV)
    h_ref, h_got = h.clone(), h.clone()
    want = ref.add_rmsnorm(h_ref, delta, w, eps, dtype, rows=rows)
    got = ops().add_rmsnorm(h_got, delta, w, eps, dtype, rows=rows)
    assert got.shape == (3, H)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
    assert torch.equal(h_got, h) and torch.equal(h_ref, h)     # picking rows (even twice) leaves the residual alone


def test_rmsnorm_reference_vector():
    # [3,4] with weights [1,2], eps 0 -> [0.84852814, 2.2627418] (src/kernel/core/cpu.zig:193-204)
    h = torch.tensor([[3.0, 4.0]], device=DEV)
    w = torch.tensor([1.0, 2.0], device=DEV)
    got = ops().add_rmsnorm(h, None, w, 0.0, torch.float32)
    torch.testing.assert_close(got.cpu(), torch.tensor([[0.84852814, 2.2627418]]), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(7, 200), (3, 12288), (1, 17)])
def test_swiglu(dtype, T, I):
    gu = rnd(T, 2 * I, dtype=dtype, scale=2.0)
    torch.testing.assert_close(ops().swiglu(gu).float(), ref.swiglu(gu).float(), **tol(dtype))


def test_swiglu_reference_vector():
    # gate [0,1,-1], up [1,2,3] -> [0, 1.4621172, -0.8068243] (src/kernel/core/cpu.zig:233-245)
    gu = torch.tensor([[0.0, 1.0, -1.0, 1.0, 2.0, 3.0]], device=DEV)
    torch.testing.assert_close(ops().swiglu(gu).cpu(), torch.tensor([[0.0, 1.4621172, -0.8068243]]), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("n_pos,d,theta", [(128, 16, 1e4), (4096, 128, 1e6), (300, 48, 5e4)])
def test_rope_table(n_pos, d, theta):
    cos, sin = ops().rope_table(n_pos, d, theta, DEV)
    rc, rs = ref.rope_table(n_pos, d, theta, "cpu")
    # same 32-bit recipe; the device's pow may differ from the host's in the last place of inv_freq,
    # which moves the angle by at most pos * 2^-24 * inv_freq
    np.testing.assert_allclose(cos.cpu().numpy(), rc.numpy(), atol=n_pos * 1.2e-7, rtol=0)
    np.testing.assert_allclose(sin.cpu().numpy(), rs.numpy(), atol=n_pos * 1.2e-7, rtol=0)
    np.testing.assert_array_equal(cos[0].cpu().numpy(), np.ones(d // 2, dtype=np.float32))  # identity at position 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page,norm,rope", [
    (4, 2, 16, 16, True, True), (6, 1, 32, 8, True, True), (3, 3, 48, 32, True, True),
    (32, 8, 128, 16, True, True), (5, 5, 80, 4, False, True), (2, 1, 256, 16, True, False)])
@pytest.mark.parametrize("T", [11, 300])   # a few tokens; a prompt portion (bfloat16 rows then take the 16-byte kernel)
def test_qk_norm_rope_store(dtype, nq, nkv, d, page, norm, rope, T):
    n_pages, n_pos = -(-T // page) + 3, 200
    qkv = rnd(T, (nq + 2 * nkv) * d, dtype=dtype)
    qw = (1 + 0.1 * rnd(d, seed=3)) if norm else None
    kw = (1 + 0.1 * rnd(d, seed=4)) if norm else None
    cos, sin = ref.rope_table(n_pos, d, 1e4, DEV) if rope else (None, None)
    positions = torch.randint(0, n_pos, (T,), dtype=torch.int32, device=DEV)
    slots = torch.randperm(n_pages * page, device=DEV)[:T].to(torch.int32)
    kc = torch.zeros(n_pages, nkv, page, d, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    kc_ref, vc_ref, qkv_ref = kc.clone(), vc.clone(), qkv.clone()
    ref.qk_norm_rope_store(qkv_ref, nq, nkv, d, qw, kw, 1e-6, cos, sin, positions, kc_ref, vc_ref, slots, page)
    ops().qk_norm_rope_store(qkv, nq, nkv, d, qw, kw, 1e-6, cos, sin, positions, kc, vc, slots, page)
    torch.testing.assert_close(qkv[:, :nq * d].float(), qkv_ref[:, :nq * d].float(), **tol(dtype))
    torch.testing.assert_close(kc.float(), kc_ref.float(), **tol(dtype))
    torch.testing.assert_close(vc.float(), vc_ref.float(), rtol=0, atol=0)
    # a reader of another layer's cache rotates q only and writes nothing
    q_only = qkv_ref.clone()[:, :nq * d].contiguous()
    q_in = rnd(T, nq * d, dtype=dtype, seed=9)
    q_ref = q_in.clone()
    ref.qk_norm_rope_store(q_ref, nq, nkv, d, qw, kw, 1e-6, cos, sin, positions, None, None, None, page, write_kv=False)
    before = kc.clone()
    ops().qk_norm_rope_store(q_in, nq, nkv, d, qw, kw, 1e-6, cos, sin, positions, None, None, None, page, write_kv=False)
    torch.testing.assert_close(q_in.float(), q_ref.float(), **tol(dtype))
    assert torch.equal(kc, before)


def test_rope_pair_rotation_reference_vector():
    # position 1, theta 1e4, d = 4: pairs (0,2) and (1,3) rotate by 1 and 0.01 rad (src/kernel/attention/rope.zig:145-190)
    d = 4
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]], device=DEV)
    cos, sin = ops().rope_table(4, d, 1e4, DEV)
    pos = torch.tensor([1], dtype=torch.int32, device=DEV)
    ops().qk_norm_rope_store(x, 1, 0, d, None, None, 0.0, cos, sin, pos, None, None, None, 1, write_kv=False)
    a0, a1 = 1.0, 0.01
    want = [1 * np.cos(a0) - 3 * np.sin(a0), 2 * np.cos(a1) - 4 * np.sin(a1),
            3 * np.cos(a0) + 1 * np.sin(a0), 4 * np.cos(a1) + 2 * np.sin(a1)]
    np.testing.assert_allclose(x.cpu().numpy()[0], np.array(want, dtype=np.float32), rtol=1e-6)


@pytest.mark.parametrize("xdt,wdt,odt", [(torch.float32,) * 3, (torch.bfloat16,) * 3,
                                         (torch.bfloat16, torch.bfloat16, torch.float32),
                                         (torch.bfloat16, torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("M,N,K", [(1, 301, 72), (7, 200, 96), (130, 389, 160), (64, 1000, 4096), (33, 65, 17)])
def test_linear(xdt, wdt, odt, M, N, K):
    x = rnd(M, K, dtype=xdt)
    w = rnd(N, K, dtype=wdt, scale=0.05, seed=1)
    got = ops().linear(x, w, out_dtype=odt)
    want = (x.double() @ w.double().T)
    t = dict(rtol=1e-5, atol=1e-5 * K ** 0.5 * 0.05) if odt == torch.float32 and xdt == torch.float32 else \
        (dict(rtol=1e-5, atol=1e-4) if odt == torch.float32 else dict(rtol=8e-3, atol=1e-3))
    assert got.dtype == odt
    torch.testing.assert_close(got.double(), want, **t)
    # strided input rows (a slice of a wider buffer)
    wide = rnd(M, K + 24, dtype=xdt, seed=5)
    got2 = ops().linear(wide[:, :K], w, out_dtype=odt)
    torch.testing.assert_close(got2.double(), wide[:, :K].double() @ w.double().T, **t)


def test_split_products_and_their_consumers():
    """A product split along K may come back as partial sums; each consumer that adds
    them itself must agree with the product reduced first."""
    o = ops()
    M, K = 8, 12288
    x = rnd(M, K, dtype=torch.bfloat16)
    # residual add + norm
    w = rnd(4096, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    part = o.linear(x, w, allow_partials=True)
    assert isinstance(part, o.Partials) and part.splits > 1 and tuple(part.shape) == (M, 4096)
    whole = o.linear(x, w)
    torch.testing.assert_close(part.sum(torch.float32), x.float() @ w.float().T, rtol=1e-3, atol=2e-2)
    h = rnd(M, 4096, scale=2.0, seed=2)
    nw = 1 + 0.1 * rnd(4096, seed=3)
    h1, h2 = h.clone(), h.clone()
    a = o.add_rmsnorm(h1, part, nw, 1e-6, torch.bfloat16)
    b = o.add_rmsnorm(h2, whole, nw, 1e-6, torch.bfloat16)
    # `whole` was rounded to bfloat16 first: half an ulp (2^-9 relative) of the largest update
    torch.testing.assert_close(h1, h2, rtol=0, atol=float(whole.float().abs().max()) * 2 ** -8 + 1e-3)
    torch.testing.assert_close(a.float(), b.float(), rtol=1.6e-2, atol=2e-2)
    rows = torch.tensor([5, 0], dtype=torch.int32, device=DEV)
    h3 = h.clone()
    c = o.add_rmsnorm(h3, part, nw, 1e-6, torch.bfloat16, rows=rows)
    torch.testing.assert_close(c.float(), a[[5, 0]].float(), rtol=0, atol=0)
    # SwiGLU
    wgu = rnd(2 * 1024, K, dtype=torch.bfloat16, scale=0.02, seed=4)
    pgu = o.linear(x, wgu, allow_partials=True)
    assert isinstance(pgu, o.Partials)
    torch.testing.assert_close(o.swiglu(pgu, out_dtype=torch.bfloat16).float(), o.swiglu(o.linear(x, wgu)).float(),
                               rtol=2e-2, atol=2e-2)
    # q/k norm + rotary + cache write
    nq, nkv, d, page = 8, 2, 128, 16
    wqkv = rnd((nq + 2 * nkv) * d, K, dtype=torch.bfloat16, scale=0.02, seed=5)
    pq = o.linear(x, wqkv, allow_partials=True)
    assert isinstance(pq, o.Partials)
    qw, kw = 1 + 0.1 * rnd(d, seed=6), 1 + 0.1 * rnd(d, seed=7)
    cos, sin = ref.rope_table(64, d, 1e4, DEV)
    positions = torch.arange(M, dtype=torch.int32, device=DEV) * 3
    slots = torch.arange(M, dtype=torch.int32, device=DEV) + 5
    caches = [torch.zeros(4, nkv, page, d, dtype=torch.bfloat16, device=DEV) for _ in range(4)]
    q1 = o.qk_norm_rope_store(pq, nq, nkv, d, qw, kw, 1e-6, cos, sin, positions, caches[0], caches[1], slots, page,
                              out_dtype=torch.bfloat16)
    q2 = o.qk_norm_rope_store(o.linear(x, wqkv), nq, nkv, d, qw, kw, 1e-6, cos, sin, positions, caches[2], caches[3],
                              slots, page)
    assert q1.shape == (M, nq * d)
    torch.testing.assert_close(q1.float(), q2[:, :nq * d].float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(caches[0].float(), caches[2].float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(caches[1].float(), caches[3].float(), rtol=2e-2, atol=2e-2)
    assert o.kernel_status() == 0


@pytest.mark.parametrize("M,I,K", [(1, 256, 128), (8, 3072, 4096), (33, 640, 200), (64, 1024, 512), (65, 192, 72),
                                   (300, 512, 264), (2048, 1536, 1024), (130, 64, 64)])
def test_linear_swiglu_fused_epilogue(M, I, K):
    """gate_up product with the SwiGLU in its epilogue, few tokens (weight rows on the MMA
    lanes, exchange through shared memory) and many (tokens on the lanes)."""
    o = ops()
    x = rnd(M, K, dtype=torch.bfloat16)
    wg = rnd(I, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    wu = rnd(I, K, dtype=torch.bfloat16, scale=0.05, seed=2)
    w = o.interleave_gate_up(wg, wu)
    assert torch.equal(w[:64], wg[:64]) and torch.equal(w[64:128], wu[:64]) and torch.equal(w[128:192], wg[64:128])
    got = o.linear_swiglu(x, w)
    g = x.float() @ wg.float().T
    u = x.float() @ wu.float().T
    want = g / (1 + torch.exp(-g)) * u
    assert got.shape == (M, I) and got.dtype == torch.bfloat16
    torch.testing.assert_close(got.float(), want, rtol=1.6e-2, atol=2e-3 * K ** 0.5 * 0.05 + 1e-3)
    # the unfused route (product, then the SwiGLU kernel on the interleaved columns) agrees
    unfused = o.swiglu(o.linear(x, w), interleave=64)
    torch.testing.assert_close(unfused.float(), want, rtol=2e-2, atol=2e-3 * K ** 0.5 * 0.05 + 2e-3)
    assert o.kernel_status() == 0


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 1000, 264), (1000, 4096, 512), (2048, 768, 4096),
                                   (2100, 389 * 2, 160)])
def test_linear_with_the_kernel_for_cta_pairs(M, N, K):
    """The product on pairs of CTAs (tcgen05 cta_group::2: tiles of 256 tokens x 256 weight rows, each
    CTA loading half of the weight rows), which is off unless asked for: plain and with the SwiGLU
    epilogue, with ragged last tiles on every side, bfloat16 and float32 results."""
    o = ops()
    x = rnd(M, K, dtype=torch.bfloat16)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    want = x.double() @ w.double().T
    before = o.gemm_pair_kernel(True)
    try:
        got = o.linear(x, w)
        got32 = o.linear(x, w, out_dtype=torch.float32)
        if N % 128 == 0:
            wg, wu = w[:N // 2].contiguous(), w[N // 2:].contiguous()
            act = o.linear_swiglu(x, o.interleave_gate_up(wg, wu))
    finally:
        o.gemm_pair_kernel(before)
    torch.testing.assert_close(got.double(), want, rtol=8e-3, atol=1e-3)
    torch.testing.assert_close(got32.double(), want, rtol=1e-5, atol=1e-4)
    single = o.linear(x, w, out_dtype=torch.float32)
    torch.testing.assert_close(got32, single, rtol=1e-5, atol=1e-4)
    if N % 128 == 0:
        g, u = want[:, :N // 2].float(), want[:, N // 2:].float()
        torch.testing.assert_close(act.float(), g / (1 + torch.exp(-g)) * u, rtol=1.6e-2, atol=2e-3 * K ** 0.5 * 0.05 + 1e-3)
    assert o.kernel_status() == 0


def _paged_case(dtype, nq, nkv, d, page, q_lens, ctx_lens, seed=0):
    """Random requests laid out in shuffled pages; returns the kernel's arguments."""
    o = ops()
    rng = np.random.RandomState(seed)
    n = len(q_lens)
    kv_lens = [c + q for c, q in zip(ctx_lens, q_lens)]
    blocks = [-(-kv // page) for kv in kv_lens]
    n_pages = sum(blocks) + 3
    perm = rng.permutation(n_pages)
    W = max(blocks)
    bt = -np.ones((n, W), dtype=np.int32)
    p = 0
    for i, b in enumerate(blocks):
        bt[i, :b] = perm[p:p + b]
        p += b
    kc = rnd(n_pages, nkv, page, d, dtype=dtype, seed=seed + 1)
    vc = rnd(n_pages, nkv, page, d, dtype=dtype, seed=seed + 2)
    T = sum(q_lens)
    q = rnd(T, nq * d + 8, dtype=dtype, seed=seed + 3)[:, :nq * d]   # strided rows
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    tr = o.attention_tile_rows()
    tseq = [i for i, ql in enumerate(q_lens) for _ in range(-(-ql // tr))]
    tq0 = [t * tr for ql in q_lens for t in range(-(-ql // tr))]
    dev = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    return dict(q=q, k_cache=kc, v_cache=vc, block_tables=dev(bt), cu_q=dev(cu), kv_lens=dev(kv_lens),
                tile_seq=dev(tseq), tile_q0=dev(tq0), num_heads=nq, num_kv_heads=nkv, head_dim=d, page_size=page)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page,window", [
    (4, 2, 16, 16, None), (6, 1, 32, 8, None), (3, 3, 48, 32, None), (8, 2, 128, 16, None),
    (5, 1, 80, 4, 7), (4, 4, 64, 16, 33), (2, 1, 256, 16, None), (4, 2, 112, 16, 20)])
def test_paged_attention(dtype, nq, nkv, d, page, window):
    q_lens = [1, 37, 2, 1, 19]
    ctx_lens = [70, 0, 15, 0, 48]
    args = _paged_case(dtype, nq, nkv, d, page, q_lens, ctx_lens)
    scale = float(1 / np.sqrt(d))
    got = ops().paged_attention(window=window, scale=scale, **args)
    want = ref.paged_attention(window=window, scale=scale, **args)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_finds_one_far_key(dtype):
    """One key among hundreds is made to stand out; the output must be its value.
    A wrong page, a wrong offset or a missed tile would pick another value."""
    nq, nkv, d, page = 4, 2, 64, 16
    args = _paged_case(dtype, nq, nkv, d, page, q_lens=[1, 3], ctx_lens=[700, 300], seed=5)
    for seq, far in ((0, 123), (1, 17)):
        pg = int(args["block_tables"][seq, far // page])
        args["k_cache"][pg, :, far % page, :] = 0
        args["k_cache"][pg, :, far % page, 0] = 60.0
    q = torch.zeros(4, nq * d, dtype=dtype, device=DEV)
    q.view(4, nq, d)[:, :, 0] = 60.0
    args["q"] = q
    got = ops().paged_attention(window=None, scale=float(1 / np.sqrt(d)), **args).float().view(4, nq, d)
    for t, (seq, far) in enumerate([(0, 123), (1, 17), (1, 17), (1, 17)]):
        pg = int(args["block_tables"][seq, far // page])
        for h in range(nq):
            torch.testing.assert_close(got[t, h], args["v_cache"][pg, h // 2, far % page].float(), rtol=2e-2, atol=2e-2)


def test_paged_attention_ignores_stale_page_contents():
    """Keys beyond a request's length in its last page, and pages of other requests,
    hold huge values; none may leak into the result."""
    dtype = torch.float32
    args = _paged_case(dtype, 4, 2, 32, 16, q_lens=[5], ctx_lens=[6], seed=8)
    clean = ops().paged_attention(window=None, scale=0.17, **args).clone()
    pg_last = int(args["block_tables"][0, 0])
    args["k_cache"][pg_last, :, 11:, :] = 1e4
    args["v_cache"][pg_last, :, 11:, :] = 1e4
    used = set(args["block_tables"][0].tolist())
    for pg in range(args["k_cache"].shape[0]):
        if pg not in used:
            args["k_cache"][pg] = 1e4
            args["v_cache"][pg] = -1e4
    dirty = ops().paged_attention(window=None, scale=0.17, **args)
    assert torch.equal(clean, dirty)


def _as_step(args, q_lens, ctx_lens):
    """The request arrays the dispatching `ops.attention` reads from a StepContext."""
    from types import SimpleNamespace
    pf = ops().attention_prefill_tile_rows()
    dev = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    dec = [i for i, ql in enumerate(q_lens) if ql == 1]
    tiles = [(i, t * pf) for i, ql in enumerate(q_lens) if ql > 1 for t in range(-(-ql // pf))]
    return SimpleNamespace(cu_q=args["cu_q"], kv_lens=args["kv_lens"], tile_seq=args["tile_seq"], tile_q0=args["tile_q0"],
                           dec_seq=dev(dec), pf_tile_seq=dev([i for i, _ in tiles]), pf_tile_q0=dev([t for _, t in tiles]),
                           n_dec=len(dec), n_pf_tiles=len(tiles), max_kv_len=max(c + q for c, q in zip(ctx_lens, q_lens)))


@pytest.mark.parametrize("nq,nkv,d,page,window", [
    (8, 2, 128, 16, None), (32, 8, 128, 16, None), (6, 1, 64, 8, None), (5, 5, 64, 32, None), (4, 2, 128, 16, 100),
    (16, 1, 128, 16, None), (6, 2, 64, 4, 37), (2, 1, 256, 16, None), (48, 3, 128, 16, None)])
@pytest.mark.parametrize("q_lens,ctx_lens", [
    ([1, 1, 1, 1], [0, 63, 64, 700]),                  # decode only, lengths around a tile's edge
    ([300, 17], [0, 130]),                             # prompt portions only, one across several query tiles
    ([1, 37, 2, 1, 129, 1], [70, 0, 15, 0, 48, 255]),  # mixed
    ([700, 3], [333, 60]),                             # a long portion behind a long context: many key tiles per query tile
])
@pytest.mark.parametrize("prefill_kernel", ["mma", "tcgen05"])
def test_tensor_core_attention(nq, nkv, d, page, window, q_lens, ctx_lens, prefill_kernel, monkeypatch):
    """The bfloat16 tensor-core kernels (prefill tiles by mma.sync or by tcgen05 with S and O
    in tensor memory, and split-key decode) through the dispatcher, against the plain reference."""
    if prefill_kernel == "tcgen05" and (d != 128 or max(q_lens) == 1):
        pytest.skip("the tcgen05 prefill kernel takes head size 128")
    monkeypatch.setattr(ops(), "PREFILL_ATTENTION", prefill_kernel)
    args = _paged_case(torch.bfloat16, nq, nkv, d, page, q_lens, ctx_lens, seed=2)
    step = _as_step(args, q_lens, ctx_lens)
    scale = float(1 / np.sqrt(d))
    got = ops().attention(args["q"], args["k_cache"], args["v_cache"], args["block_tables"], step, nq, nkv, d, page,
                          window, scale)
    want = ref.paged_attention(window=window, scale=scale, **args)
    torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2, atol=1.5e-2)
    # every split count gives the same answer up to rounding
    for forced in (1, 3, 32):
        step.max_kv_len = 64 * forced
        again = ops().attention(args["q"], args["k_cache"], args["v_cache"], args["block_tables"], step, nq, nkv, d,
                                page, window, scale)
        torch.testing.assert_close(again.float(), want.float(), rtol=1.6e-2, atol=1.5e-2)


@pytest.mark.parametrize("nq,nkv,d,page,window", [(32, 8, 128, 16, None), (6, 1, 64, 8, 37), (8, 1, 128, 32, None),
                                                   (2, 1, 256, 16, None), (5, 5, 64, 16, 200)])
def test_decode_attention_both_tile_forms(nq, nkv, d, page, window):
    """Groups of at most 8 query heads take the tile with the keys on the MMA's rows; the form with
    the heads on the rows (which larger groups use) must give the same, and both the reference; each
    with the keys and values brought by TMA page boxes and by cp.async."""
    o = ops()
    ctx_lens = [0, 15, 16, 63, 64, 65, 700, 1300]
    q_lens = [1] * len(ctx_lens)
    args = _paged_case(torch.bfloat16, nq, nkv, d, page, q_lens, ctx_lens, seed=6)
    step = _as_step(args, q_lens, ctx_lens)
    scale = float(1 / np.sqrt(d))
    want = ref.paged_attention(window=window, scale=scale, **args)
    outs = {}
    try:
        for tma in (True, False):
            o.decode_tma(tma)
            for on in (True, False):
                o.decode_transposed_tile(on)
                for forced in (1, 5):
                    step.max_kv_len = 64 * forced
                    got = o.attention(args["q"], args["k_cache"], args["v_cache"], args["block_tables"], step, nq, nkv, d,
                                      page, window, scale)
                    torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2, atol=1.5e-2)
                    outs[(tma, on, forced)] = got.float()
    finally:
        o.decode_transposed_tile(True)
        o.decode_tma(1)
    torch.testing.assert_close(outs[(True, True, 5)], outs[(True, False, 5)], rtol=1.6e-2, atol=4e-3)
    assert torch.equal(outs[(True, True, 5)], outs[(False, True, 5)]), "the same tile read from TMA boxes and from cp.async rows differs"
    o.require_kernel_status_ok("decode attention")


@pytest.mark.parametrize("nq,nkv,d,page,window,norm,rope,partial", [
    (32, 8, 128, 16, None, True, True, True), (8, 2, 128, 16, None, True, True, False), (6, 1, 64, 8, 50, True, True, False),
    (5, 5, 64, 32, None, False, True, False), (16, 1, 128, 16, None, True, False, False), (2, 1, 256, 16, None, True, True, False)])
def test_fused_decode_attention_equals_the_two_kernels(nq, nkv, d, page, window, norm, rope, partial):
    """q/k norm + rotary + cache write + attention in one kernel against the same done by
    qk_norm_rope_store followed by the decode attention: outputs and cache contents agree."""
    o = ops()
    ctx_lens = [0, 1, 63, 64, 700, 129, 15, 300]       # the token is the first, crosses tiles, ...
    q_lens = [1] * len(ctx_lens)
    args = _paged_case(torch.bfloat16, nq, nkv, d, page, q_lens, ctx_lens, seed=4)
    step = _as_step(args, q_lens, ctx_lens)
    T = len(q_lens)
    step.n_seqs = T
    step.positions = torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)
    slots = torch.tensor([int(args["block_tables"][i, c // page]) * page + c % page for i, c in enumerate(ctx_lens)],
                         dtype=torch.int32, device=DEV)
    width = (nq + 2 * nkv) * d
    if partial:
        x = rnd(T, 4096, dtype=torch.bfloat16, seed=8)
        w = rnd(width, 4096, dtype=torch.bfloat16, scale=0.02, seed=9)
        qkv = o.linear(x, w, allow_partials=True)
        assert isinstance(qkv, o.Partials)
        qkv2 = o.Partials(qkv.data.clone())
    else:
        qkv = rnd(T, width, dtype=torch.bfloat16, seed=8)
        qkv2 = qkv.clone()
    qw = (1 + 0.1 * rnd(d, seed=3)) if norm else None
    kw = (1 + 0.1 * rnd(d, seed=4)) if norm else None
    cos, sin = ref.rope_table(1024, d, 1e4, DEV) if rope else (None, None)
    scale = float(1 / np.sqrt(d))
    k1, v1 = args["k_cache"].clone(), args["v_cache"].clone()
    k2, v2 = args["k_cache"].clone(), args["v_cache"].clone()
    assert o.decode_fused_ok(torch.bfloat16, nq, nkv, d, step)
    fused = o.attention_decode_fused(qkv, nq, nkv, d, qw, kw, 1e-6, cos, sin, k1, v1, slots, args["block_tables"], step,
                                     page, window, scale)
    q = o.qk_norm_rope_store(qkv2, nq, nkv, d, qw, kw, 1e-6, cos, sin, step.positions, k2, v2, slots, page,
                             out_dtype=torch.bfloat16)
    two = o.attention(q, k2, v2, args["block_tables"], step, nq, nkv, d, page, window, scale)
    assert torch.equal(k1, k2) and torch.equal(v1, v2), "the fused kernel wrote other keys or values"
    torch.testing.assert_close(fused.float(), two.float(), rtol=1.6e-2, atol=1e-2)


def test_tensor_core_attention_finds_one_far_key_and_ignores_stale_pages():
    nq, nkv, d, page = 8, 2, 128, 16
    q_lens, ctx_lens = [1, 200, 1], [900, 100, 33]
    args = _paged_case(torch.bfloat16, nq, nkv, d, page, q_lens, ctx_lens, seed=5)
    used = set(int(p) for p in args["block_tables"].flatten().tolist() if p >= 0)
    for pg in range(args["k_cache"].shape[0]):
        if pg not in used:
            args["k_cache"][pg] = 300.0
            args["v_cache"][pg] = -300.0
    last = int(args["block_tables"][2, 33 // page])            # request 2 holds 34 keys: offsets 2.. of its last page are stale
    args["k_cache"][last, :, 2:, :] = 300.0
    args["v_cache"][last, :, 2:, :] = -300.0
    far = {0: 123, 1: 17, 2: 5}
    for seq, pos in far.items():
        pg = int(args["block_tables"][seq, pos // page])
        args["k_cache"][pg, :, pos % page, :] = 0
        args["k_cache"][pg, :, pos % page, 0] = 40.0
    T = sum(q_lens)
    q = torch.zeros(T, nq * d, dtype=torch.bfloat16, device=DEV)
    q.view(T, nq, d)[:, :, 0] = 40.0
    args["q"] = q
    step = _as_step(args, q_lens, ctx_lens)
    got = ops().attention(q, args["k_cache"], args["v_cache"], args["block_tables"], step, nq, nkv, d, page, None,
                          float(1 / np.sqrt(d))).float().view(T, nq, d)
    seq_of = [0] + [1] * 200 + [2]
    for t in (0, 1, 100, 200, 201):
        seq = seq_of[t]
        pg = int(args["block_tables"][seq, far[seq] // page])
        for h in range(nq):
            torch.testing.assert_close(got[t, h], args["v_cache"][pg, h // 4, far[seq] % page].float(), rtol=2e-2, atol=3e-2)


def test_attention_refuses_what_it_cannot_do():
    o = ops()
    args = _paged_case(torch.float32, 2, 1, 272, 16, [1], [3])
    with pytest.raises(o.KernelError, match="head_dim"):
        o.paged_attention(window=None, scale=1.0, **args)


@pytest.mark.parametrize("R,V", [(1, 301), (5, 151936), (64, 1000)])
def test_argmax_first_maximum_wins(R, V):
    logits = rnd(R, V)
    logits[0, 7] = logits[0, V - 1] = 100.0   # a tie: the lower id wins (src/sampling/sampler.zig:93-105)
    got = ops().argmax(logits)
    want = torch.stack([torch.tensor(int(np.argmax(row))) for row in logits.cpu().numpy()]).to(torch.int32)
    assert torch.equal(got.cpu(), want)
    assert int(got[0]) == 7


@pytest.mark.parametrize("M,N,K,fused", [(1, 301, 72, True), (8, 5000, 256, True), (64, 1000, 136, True),
                                           (128, 389, 64, True), (3, 151936, 64, True), (16, 20000, 1024, True), (16, 4133, 4096, False),
                                           (130, 389, 64, False), (8, 256, 4096, False)])
def test_argmax_in_the_output_heads_epilogue(M, N, K, fused):
    """The head's product leaves one candidate per 32 weight rows and a small kernel picks among
    them: the ids are those of the argmax kernel over the same logits (first maximum, NaN as -inf),
    the logits are bit for bit the plain product's.  More than 128 rows, or a K that is split, take
    the two kernels instead (src/sampling/sampler.zig:93-105)."""
    o = ops()
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.1)
    w[N - 1] = w[5] = (x[0].float() * 4).to(torch.bfloat16)      # a tie inside one warp's rows or across tiles
    if N > 200:
        w[200] = w[5]
    w[9] = float("nan")                                           # a row of NaN logits never wins
    x[M - 1] = 0                                                  # a row of zeros: every finite logit ties, id 0 wins
    from zinfer_b200 import profiling
    with profiling.profile() as prof:
        logits, ids = o.linear_argmax(x, w)
    classes = {c["class"] for c in prof.summary()["classes"]}
    assert ("argmax (candidates)" in classes) == fused and ("argmax" in classes) != fused
    plain = o.linear(x, w, out_dtype=torch.float32)
    assert torch.equal(logits.nan_to_num(nan=-7.0), plain.nan_to_num(nan=-7.0))
    assert torch.equal(ids, o.argmax(plain))
    assert int(ids[0]) == 5 or M == 1                             # (with one row, row 0 is the row of zeros)
    assert int(ids[M - 1]) == 0
    # all logits negative, and -0 beside +0
    xn = torch.ones((M, K), dtype=torch.bfloat16, device="cuda")
    wn = -rnd(N, K, dtype=torch.bfloat16, scale=0.1).abs() - 0.01
    wn[N // 2] = 0.0
    wn[3] = -0.0
    logits, ids = o.linear_argmax(xn, wn)
    assert torch.equal(ids, o.argmax(logits)) and int(ids[0]) == 3
    o.require_kernel_status_ok("linear_argmax")


def test_a_wait_that_runs_out_is_reported_not_survived_silently():
    """The tensor-core kernels bound every wait; when one runs out they record a code in a device
    word and return.  Here a one-CTA kernel waits on a barrier nobody arrives at, with a limit of a
    few thousand tries: it returns normally, the word holds the code, the check that the engine,
    the replay program and the benchmark make raises, and the library works on afterwards."""
    o = ops()
    assert o.kernel_status() == 0
    o.selftest_wait_runs_out(code=77, tries=4096)
    torch.cuda.synchronize()
    with pytest.raises(o.KernelError, match="code 77"):
        o.require_kernel_status_ok("test")
    assert o.kernel_status() == 0, "reading the status clears it"
    x, w = rnd(8, 4096, dtype=torch.bfloat16), rnd(256, 4096, dtype=torch.bfloat16, scale=0.05)
    got = o.linear(x, w, out_dtype=torch.float32)
    torch.testing.assert_close(got, x.float() @ w.float().T, rtol=1e-3, atol=1e-2)
    o.require_kernel_status_ok("after")
    with pytest.raises(o.KernelError):
        o.selftest_wait_runs_out(code=0)
