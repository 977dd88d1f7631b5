"""The native step builder (csrc/host_runtime.cpp: zi_step_build) against a plain
re-derivation of every array it fills, for random mixes of prompt portions and single
tokens over two cache groups (one with a window), uncaptured and in a padded bucket."""
import random

import numpy as np
import pytest
import torch

from zinfer_b200.cache import CacheManager
from zinfer_b200.engine import StepEntry, build_step
from zinfer_b200.engine.batch import StaticStepBuffers
from zinfer_b200.parts import KVCacheNeed


def _manager(page=4, pages=400, window=9):
    return CacheManager({"full": KVCacheNeed(2, 16, None), "win": KVCacheNeed(1, 16, window)}, ["s"], page, pages, 16)


def _expected(m, entries, tile_rows, pf_rows):
    ps = m.page_size
    q = [len(e.tokens) for e in entries]
    ctx = [m.length(e.request_id) for e in entries]
    cu = np.concatenate([[0], np.cumsum(q)])
    exp = dict(
        token_ids=np.concatenate([np.maximum(np.asarray(e.tokens), 0) for e in entries]),
        positions=np.concatenate([np.arange(c, c + n) for c, n in zip(ctx, q)]),
        cu_q=cu, kv_lens=np.asarray(ctx) + np.asarray(q),
        state_slots=np.asarray([m.requests[e.request_id].state_slot for e in entries]),
        logit_rows=np.asarray([cu[i] + w for i, e in enumerate(entries) for w in e.want], dtype=np.int64),
        dec_seq=np.asarray([i for i, n in enumerate(q) if n == 1], dtype=np.int64),
        tile_seq=np.asarray([i for i, n in enumerate(q) for _ in range(-(-n // tile_rows))]),
        tile_q0=np.asarray([t * tile_rows for n in q for t in range(-(-n // tile_rows))]))
    pf = [(i, t * pf_rows) for i, n in enumerate(q) if n > 1 for t in range(-(-n // pf_rows))]
    pf.sort(key=lambda it: -(ctx[it[0]] + min(q[it[0]], it[1] + pf_rows)))
    exp["pf_tile_seq"], exp["pf_tile_q0"] = np.asarray([i for i, _ in pf], dtype=np.int64), np.asarray([t for _, t in pf], dtype=np.int64)
    for gi in range(len(m.groups)):
        tables = [m.block_table(e.request_id, gi) for e in entries]
        exp[f"slots{gi}"] = np.concatenate([[tables[i][p // ps] * ps + p % ps for p in range(c, c + n)]
                                            for i, (c, n) in enumerate(zip(ctx, q))])
        exp[f"tables{gi}"] = tables
    return exp


@pytest.mark.parametrize("seed", range(6))
def test_mixed_steps_fill_every_array(seed):
    rng = random.Random(seed)
    m = _manager()
    live = {}
    for step in range(12):
        for _ in range(rng.randint(0, 2)):
            if len(live) < 6:
                rid = f"r{step}_{len(live)}_{rng.randrange(1000)}"
                m.add_request(rid)
                live[rid] = 0
        if not live:
            continue
        chosen = rng.sample(sorted(live), rng.randint(1, len(live)))
        entries = []
        for rid in chosen:
            n = 1 if rng.random() < 0.5 else rng.randint(2, 23)
            toks = [rng.randrange(1000) for _ in range(n)]
            src = None
            if n == 1 and rng.random() < 0.3:
                toks, src = [-1], rng.randrange(8)
            want = sorted(rng.sample(range(n), rng.randint(0, min(n, 3))))
            entries.append(StepEntry(rid, toks, want, token_src=src))
            m.reserve(rid, n)
        ctx = build_step(m, entries, "cpu", tile_rows=8, pin=False, pf_tile_rows=16)
        exp = _expected(m, entries, 8, 16)
        for name in ("token_ids", "positions", "cu_q", "kv_lens", "state_slots", "dec_seq", "tile_seq", "tile_q0",
                     "pf_tile_seq", "pf_tile_q0"):
            assert getattr(ctx, name).tolist() == exp[name].tolist(), name
        assert (ctx.logit_rows.tolist() if ctx.logit_rows is not None else []) == exp["logit_rows"].tolist()
        assert ctx.n_dec == len(exp["dec_seq"]) and ctx.n_pf_tiles == len(exp["pf_tile_seq"])
        assert ctx.n_seqs == len(entries) and ctx.n_tokens == len(exp["token_ids"]) and ctx.all_decode == all(len(e.tokens) == 1 for e in entries)
        assert ctx.ctx_lens == [m.length(e.request_id) for e in entries] and ctx.max_kv_len == int(exp["kv_lens"].max())
        patches = [(int(exp["cu_q"][i]), e.token_src) for i, e in enumerate(entries) if e.token_src is not None]
        assert ctx.n_patch == len(patches)
        if patches:
            assert list(zip(ctx.patch_dst.tolist(), ctx.patch_src.tolist())) == patches
        for gi, g in enumerate(ctx.kv_groups):
            assert g.slot_mapping.tolist() == exp[f"slots{gi}"].tolist()
            W = g.block_tables.shape[1]
            assert W == max(1, max(len(t) for t in exp[f"tables{gi}"]))
            for i, t in enumerate(exp[f"tables{gi}"]):
                assert g.block_tables[i].tolist() == t + [-1] * (W - len(t))
        for e in entries:
            m.commit(e.request_id, len(e.tokens))
            live[e.request_id] += len(e.tokens)
            if rng.random() < 0.15:
                m.free_request(e.request_id)
                del live[e.request_id]
        m.check()


def test_a_bucket_is_padded_with_requests_that_touch_nothing():
    m = _manager(page=4)
    for rid, n in (("a", 9), ("b", 3)):
        m.add_request(rid)
        m.reserve(rid, n)
        m.commit(rid, n)
    entries = [StepEntry("a", [7], [0]), StepEntry("b", [-1], [0], token_src=1)]
    for e in entries:
        m.reserve(e.request_id, 1)
    static = StaticStepBuffers(4, 5, "cpu", max_kv_len=20)
    ctx = build_step(m, entries, "cpu", tile_rows=8, static=static, pf_tile_rows=16)
    assert ctx.n_seqs == 4 and ctx.n_tokens == 4 and ctx.n_dec == 4 and ctx.max_kv_len == 20
    assert ctx.token_ids.tolist() == [7, 0, 0, 0] and ctx.positions.tolist() == [9, 3, 0, 0]
    assert ctx.kv_lens.tolist() == [10, 4, 1, 1] and ctx.cu_q.tolist() == [0, 1, 2, 3, 4]
    assert ctx.logit_rows.tolist() == [0, 1, 2, 3] and ctx.dec_seq.tolist() == [0, 1, 2, 3]
    assert ctx.patch_dst.tolist() == [1, -1, -1, -1] and ctx.patch_src.tolist()[0] == 1 and ctx.n_patch == 1
    full = ctx.kv_groups[0]
    assert full.block_tables.shape == (4, 5)
    assert full.block_tables[0].tolist()[:3] == m.block_table("a", 0) and full.block_tables[2].tolist() == [-1] * 5
    assert full.slot_mapping.tolist()[2:] == [-1, -1]            # the padding rows write no key
    # the same bucket again: the layout (and so every address a captured graph holds) is unchanged
    again = build_step(m, entries[:1], "cpu", tile_rows=8, static=static, pf_tile_rows=16)
    assert again.token_ids.data_ptr() == ctx.token_ids.data_ptr() and again.kv_lens.tolist() == [10, 1, 1, 1]
    # a request that has outgrown the bucket's tables is refused
    m.commit("a", 1)
    m.reserve("a", 12)
    m.commit("a", 12)
    m.reserve("a", 1)
    with pytest.raises(RuntimeError, match="longer than its bucket"):
        build_step(m, [StepEntry("a", [1], [0])], "cpu", tile_rows=8, static=static, pf_tile_rows=16)


def test_a_token_in_a_page_already_given_back_is_refused():
    m = CacheManager({"win": KVCacheNeed(1, 16, 4)}, [], 4, 16, 2)
    m.add_request("a")
    m.reserve("a", 12)
    m.commit("a", 12)       # the window has passed the first pages
    assert m.block_table("a", 0)[0] == -1
    m.reserve("a", 1)
    ctx = build_step(m, [StepEntry("a", [5], [0])], "cpu", tile_rows=8, pin=False)
    assert ctx.kv_groups[0].block_tables[0].tolist()[0] == -1 and ctx.kv_groups[0].slot_mapping.tolist()[0] >= 0
