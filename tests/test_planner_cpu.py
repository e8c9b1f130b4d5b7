"""The split-K planner of the PAM matrix product, queried without a GPU (it assumes a 148-SM device
when none is present).  The expected splits for the DeiT-tiny linear-layer products are the ones an
exhaustive tile x split sweep on a B200 measured fastest (within 1 %); pinning them here keeps a
change of the cost model from silently moving the benchmark's products off their optimum."""
import pytest

from pam_b200 import _lib

TOKENS = 12608


@pytest.fixture(scope="module")
def lib():
    return _lib.lib()


@pytest.mark.parametrize("M,N,K,split", [
    (TOKENS, 576, 192, 1), (TOKENS, 192, 576, 2), (192, 576, TOKENS, 43),        # 192 -> 576: forward, dX, dW
    (TOKENS, 192, 192, 1), (192, 192, TOKENS, 64),                              # 192 -> 192
    (TOKENS, 768, 192, 1), (TOKENS, 192, 768, 2), (192, 768, TOKENS, 32),        # 192 -> 768 and 768 -> 192
    (768, 192, TOKENS, 32),
])
def test_deit_products_keep_their_measured_best_split(lib, M, N, K, split):
    assert lib.pamk_matmul_auto_split(1, M, N, K) == split


@pytest.mark.parametrize("M,N,K,split", [
    (10000, 512, 4096, 6),     # 316 tiles of 128 x 128 on 296 slots: 1.07 waves unsplit (measured 1.88 -> 1.52 ms)
    (4096, 512, 10000, 8),     # the input gradient of the same projection (1.58 -> 1.51 ms)
    (2048, 3072, 2048, 3),     # 384 tiles: 1.3 waves unsplit (1.11 -> 0.97 ms)
    (4096, 10000, 512, 1),     # 8.5 waves: nothing to gain
])
def test_products_of_one_to_two_waves_are_split_to_shorten_the_last_wave(lib, M, N, K, split):
    assert lib.pamk_matmul_auto_split(1, M, N, K) == split


@pytest.mark.parametrize("batch,M,N,K,tile", [
    (1, 16384, 16384, 16384, 128), (1, 4096, 4096, 4096, 128),   # large squares
    (1, 4096, 512, 512, 128), (1, 10000, 512, 4096, 128),        # transformer products: large tile, K ranges
    (1, TOKENS, 192, 192, 64), (1, TOKENS, 576, 192, 64),        # DeiT-tiny layers: 197 x 3 tiles of 64 fill the SMs
    (192, 197, 197, 64, 32),                                     # its score products: 224 x 224 instead of 256 x 256 padded
    (512, 32, 32, 128, 32),                                      # attention over 32 tokens
    (8, 160, 197, 64, 32),                                       # a launch that leaves most SMs empty (21.6 -> 9.4 us)
])
def test_tile_choices_that_sweeps_measured_best(lib, batch, M, N, K, tile):
    assert lib.pamk_test_set_tile_policy(0) == 0
    assert lib.pamk_test_planned_tile(batch, M, N, K) == tile


def test_planner_basic_properties(lib):
    # large outputs fill the GPU without a split; tiny K is never split; empty problems do not divide by zero
    assert lib.pamk_matmul_auto_split(1, 4096, 4096, 4096) == 1
    assert lib.pamk_matmul_auto_split(1, 64, 64, 16) == 1
    assert lib.pamk_matmul_auto_split(1, 0, 64, 64) == 1 and lib.pamk_matmul_auto_split(1, 64, 64, 0) == 1
    # a weight gradient over many tokens is split for the exact-gradient product as well
    assert lib.pamk_matmul_bwd_auto_split(1, 192, 576, TOKENS) > 8
    # the split never leaves a range with fewer than four slabs of 8
    for K in (32, 64, 200, 1000, 5000):
        s = lib.pamk_matmul_auto_split(1, 64, 64, K)
        assert s == 1 or K / s >= 32
    # scratch size is the split times the output
    assert lib.pamk_matmul_workspace_bytes(2, 3, 5, 4) == 2 * 3 * 5 * 4 * 4
