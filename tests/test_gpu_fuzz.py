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


@pytest.mark.parametrize("Kdim", [8, 16, 20, 24, 32, 100])
@pytest.mark.parametrize("policy", [0, 1, 2])
@pytest.mark.parametrize("delta_l", [True, False])
def test_exact_gradient_below_offset_one_against_oracle(oracle, Kdim, policy, delta_l):
    """Offsets below one make the slope of a zero-padded K-tail term -inf for outputs whose D has a small
    mantissa: the reference's kernel pads K to a multiple of 32 (pam/cuda_kernels.cu:795-809) and so turns
    those outputs into NaN exactly when K is not a multiple of 32 - on every tile shape alike."""
    from pam_b200 import _lib, cuda_bindings as cb
    K = oracle.kernels()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(Kdim * 10 + policy)
    M, N = 70, 45
    A = torch.randn(M, Kdim, generator=g)
    B = torch.randn(Kdim, N, generator=g)
    D = torch.randn(M, N, generator=g)
    D.view(-1)[::5] = 1.0 + 2.0 ** -20                      # small mantissas
    _lib.check(_lib.lib().pamk_test_set_tile_policy(policy), "tile policy")
    try:
        for offset in (0.97, 0.9):
            got = cb._matmul_bwd(A.to(dev), B.to(dev), D.to(dev), delta_l, offset, 2, split_k=1)
            want = K.pam_matmul_bwd(A, B, D, True, True, delta_l, offset)
            assert_bits_equal(got, want, f"exact gradient, K={Kdim}, offset={offset}")
            assert bool(want.isnan().any()) == (Kdim % 32 != 0), "NaN appears exactly when K is padded"
    finally:
        _lib.lib().pamk_test_set_tile_policy(0)


def test_tall_product_beyond_the_grid_limit(oracle):
    """More than 65535 row tiles of the small tile shapes: the product moves to the 128 x 128 tile instead of
    being refused.  Rows are sampled against the oracle."""
    from pam_b200 import cuda_bindings as cb
    K = oracle.kernels()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(5)
    M, N, Kdim = 65536 * 64 + 100, 10, 12                   # 4.19 M rows: beyond 65535 tiles of 64 (and of 32)
    A = torch.randn(M, Kdim, generator=g, device=dev)
    B = torch.randn(Kdim, N, generator=g, device=dev)
    got = cb._matmul(0, A, B, 1.0, 2, split_k=1)
    rows = torch.cat([torch.arange(0, 300, device=dev), torch.arange(M - 300, M, device=dev),
                      torch.randint(0, M, (400,), generator=g, device=dev)])
    want = K.pam_matmul_fwd(A[rows].cpu(), B.cpu(), True, True, 1.0)
    assert_bits_equal(got[rows], want, "sampled rows of the tall product")
