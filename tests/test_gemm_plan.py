"""The host-side plans of the kernels (the matrix product: which side the tokens go on, the N
tile, the K split; the sampling kernel: CTAs per row): decisions only, no GPU.  The library is built by nvcc on first use."""
import ctypes
import shutil

import pytest


@pytest.fixture(scope="module")
def plan():
    if shutil.which("nvcc") is None:
        pytest.skip("no nvcc to build the kernel library with")
    from zinfer_b200 import ops

    lib = ops.lib()

    def f(M, N, K, sms=148):
        out = (ctypes.c_int * 3)()
        need = lib.zi_gemm_tcgen05_plan(M, N, K, sms, out)
        return {"swap": out[0], "BN": out[1], "splits": out[2], "workspace": int(need)}

    return f


def test_few_tokens_put_the_weight_on_the_lanes_and_split_k(plan):
    for M in (1, 8, 64, 65, 128):
        p = plan(M, 6144, 4096)
        assert p["swap"] == 1 and p["BN"] in (16, 32, 64, 128) and M <= p["BN"] < 2 * max(M, 16)
        assert p["splits"] == 4 and p["workspace"] == 4 * M * 6144 * 4      # 48 tiles x 4 = 192 CTAs in one wave
    assert plan(8, 4096, 4096)["splits"] == 8                               # 32 tiles x 8 = 256
    assert plan(8, 4096, 12288)["splits"] == 8
    assert plan(8, 24576, 4096)["splits"] == 3                              # 192 tiles: three splits fill 576 of 592 slots
    assert plan(8, 151936, 4096)["splits"] == 1                             # many waves: no split, no workspace
    assert plan(8, 151936, 4096)["workspace"] == 0


def test_many_tokens_are_left_whole_and_a_few_hundred_are_split_when_it_pays(plan):
    for N, K in [(6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288)]:
        p = plan(2048, N, K)
        assert p["swap"] == 0 and p["BN"] == 256 and p["splits"] == 1
    assert plan(129, 4096, 12288)["swap"] == 0
    assert plan(160, 4096, 12288)["splits"] > 1      # 64 tiles on 148 SMs, 192 k-blocks each
    assert plan(160, 4096, 4096)["splits"] > 1
    assert plan(256, 6144, 4096)["splits"] == 1      # 48 tiles: the partial sums would cost what the split saves
    assert plan(512, 24576, 4096)["splits"] == 1


def test_splits_never_leave_a_split_without_k_blocks(plan):
    for M in (1, 8, 64, 65, 128, 300):
        for N, K in [(128, 64), (256, 512), (1000, 264), (4096, 4096), (5120, 17408), (151936, 4096)]:
            p = plan(M, N, K)
            kb = -(-K // 64)
            assert 1 <= p["splits"] <= kb
            assert (p["workspace"] > 0) == (p["splits"] > 1)


def test_sampling_rows_share_clusters_by_the_number_of_rows():
    if shutil.which("nvcc") is None:
        pytest.skip("no nvcc to build the kernel library with")
    from zinfer_b200 import ops

    f = ops.lib().zi_sample_ctas_per_row
    assert [f(r, 148) for r in (1, 8, 18, 19, 37, 38, 64, 74, 75, 256)] == [8, 8, 8, 4, 4, 2, 2, 2, 1, 1]
    assert f(1, 4) == 4 and f(5, 4) == 1
