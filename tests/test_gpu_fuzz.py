"""Randomised differential test of the matrix-product entry points against the oracle.

Eighty seeded cases draw the shape (including sizes that are not multiples of any tile or vector
width), the batch, the memory layout of each operand, the product (PAM, true multiply, the two
exact-gradient forms), the offset, the CTA tile, an optional bias, an optional explicit split of K,
and an optional dose of special values.  Unsplit products must equal the oracle bit for bit; split
products must stay within the summation-order bound."""
import random

import pytest
import torch

from conftest import assert_bits_equal

pytestmark = pytest.mark.gpu

SPECIALS = [0.0, -0.0, 1e-40, -1e-40, 1.4e-45, 1e30, -1e30, 1e-30, float("inf"), float("-inf"), float("nan"), 3e38]


def _layout(t, transposed_storage):
    """Same values; contiguous along the last dimension, or along the one before it."""
    return t.mT.contiguous().mT if transposed_storage else t.contiguous()


@pytest.mark.parametrize("case", range(80))
def test_random_product_against_oracle(oracle, case):
    import pam_b200
    from pam_b200 import _lib, cuda_bindings as cb
    K = oracle.kernels()
    dev = torch.device("cuda", 0)
    rnd = random.Random(9000 + case)
    g = torch.Generator().manual_seed(9000 + case)
    batch = rnd.choice([1, 1, 2, 5])
    M, N = rnd.choice([1, 3, 31, 32, 33, 64, 65, 100, 197]), rnd.choice([1, 4, 30, 32, 63, 64, 96, 130, 200])
    Kdim = rnd.choice([1, 2, 7, 8, 9, 16, 64, 100, 257, 600])
    mode = rnd.choice(["pam", "pam", "pam", "std", "bwd_l", "bwd_r"])
    offset = rnd.choice([1.0, 1.0552])
    tile = rnd.choice([0, 1, 2, 3])
    split = rnd.choice([1, 1, 1, 2, 3, 8]) if mode != "std" else 1
    dims = 3 if batch > 1 or rnd.random() < 0.3 else 2
    shape = (lambda *s: (batch, *s)) if dims == 3 else (lambda *s: s)
    A = torch.randn(*shape(M, Kdim), generator=g) * rnd.choice([1.0, 1e-3, 50.0])
    B = torch.randn(*shape(Kdim, N), generator=g) * rnd.choice([1.0, 0.02])
    if rnd.random() < 0.35:
        for t in (A, B):
            flat = t.reshape(-1)
            idx = torch.randperm(flat.numel(), generator=g)[: max(1, flat.numel() // 20)]
            flat[idx] = torch.tensor(SPECIALS)[torch.arange(idx.numel()) % len(SPECIALS)]
    Ad, Bd = _layout(A.to(dev), rnd.random() < 0.5), _layout(B.to(dev), rnd.random() < 0.5)
    bias = torch.randn(N, generator=g) if mode == "pam" and rnd.random() < 0.4 else None

    lib = _lib.lib()
    _lib.check(lib.pamk_test_set_tile_policy(tile), "tile policy")
    try:
        if mode in ("pam", "std"):
            kind = 0 if mode == "pam" else 1
            got = cb._matmul(kind, Ad, Bd, offset, dims, split_k=split, bias=None if bias is None else bias.to(dev))
            want = (K.pam_matmul_fwd(A, B, True, True, offset) if mode == "pam" else K.standard_matmul(A, B))
            if bias is not None:
                want = want + bias
            terms = K.pam_matmul_fwd(A.abs(), B.abs(), True, True, offset) if mode == "pam" else None
        else:
            D = torch.randn(*shape(M, N), generator=g)
            got = cb._matmul_bwd(Ad, Bd, D.to(dev), mode == "bwd_l", offset, dims, split_k=split)
            want = K.pam_matmul_bwd(A, B, D, True, True, mode == "bwd_l", offset)
            terms = K.pam_matmul_bwd(A.abs(), B.abs(), D.abs(), True, True, mode == "bwd_l", offset)
    finally:
        lib.pamk_test_set_tile_policy(0)

    what = f"case {case}: {mode} {batch}x{M}x{N}x{Kdim} tile={tile} split={split} bias={bias is not None}"
    if split == 1:
        assert_bits_equal(got, want, what)
        return
    got = got.cpu()
    # Where the sum of the terms' magnitudes is finite no partial sum can overflow, so both orders
    # are finite and close; elsewhere (inf / NaN terms, or sums near the fp32 maximum) whether a
    # lane ends as inf or NaN depends on the order, and only "not finite" is common to both.
    ok = terms.isfinite()
    assert bool(got[ok].isfinite().all()) and bool(want[ok].isfinite().all()), what + ": finite lanes"
    bound = 4 * Kdim * 2.0 ** -24 * terms.double() + 1e-30
    assert bool(((got.double() - want.double()).abs()[ok] <= bound[ok]).all()), what
