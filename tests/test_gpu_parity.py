"""Parity of the CUDA kernels (through the C ABI) with the reference: committed fixtures generated
from the reference's own code, and the CPU oracle on seeded inputs at sizes it finishes quickly.

Bars: per-element operations bit-exact (NaN payloads aside); matrix products without split-K
bit-exact as well (same products, same k order, one accumulator); with split-K, and for values
that went through an ordinary fp32 row reduction, within a stated tolerance."""
import math

import pytest
import torch

import parity_cases as cases
from conftest import assert_bits_equal, assert_close_nan, bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pam():
    import pam_b200
    assert torch.cuda.is_available(), "gpu-marked tests need a CUDA device"
    return pam_b200


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def strict_order(pam):
    """Matrix products are compared bit for bit, so K is never split here (the split-K test
    passes its split explicitly)."""
    pam.set_strict_k_order(True)
    yield
    pam.set_strict_k_order(False)


@pytest.fixture(scope="module")
def K(oracle):
    return oracle.kernels()


@pytest.fixture(params=[1, 2, 3], ids=["tile128", "tile64", "tile32"])
def tile(request, pam):
    """Runs a matrix-product test once per CTA tile shape (the library picks one per problem)."""
    from pam_b200 import _lib
    _lib.check(_lib.lib().pamk_test_set_tile_policy(request.param), "tile policy")
    yield request.param
    _lib.lib().pamk_test_set_tile_policy(0)


SPECIALS = [0.0, -0.0, 1e-40, -1e-40, 1.4e-45, -1.4e-45, 1e30, -1e30, 1e-30, -1e-30]


def inject(t, frac, g, extra=()):
    """Overwrites a fixed fraction of entries with a cycle of special values (zeros, denormals,
    +-1e30, +-1e-30): the value distribution of the scaling-sweep configuration."""
    flat = t.reshape(-1)
    count = max(1, int(flat.numel() * frac))
    idx = torch.randperm(flat.numel(), generator=g)[:count]
    vals = torch.tensor(SPECIALS + list(extra), dtype=torch.float32)
    flat[idx] = vals[torch.arange(count) % vals.numel()]
    return t


# ---- fixtures generated from the reference -------------------------------------------------------

@pytest.mark.parametrize("oname,mode", cases.MODES)
def test_golden_mul_div(pam, golden, dev, oname, mode):
    cases.mul_div(pam, golden, dev, oname, mode)


def test_golden_broadcast(pam, golden, dev):
    cases.broadcast(pam, golden, dev, exact_sums=False)


@pytest.mark.parametrize("base", ["e", "2", "10"])
@pytest.mark.parametrize("oname,mode", cases.MODES)
def test_golden_exp_log(pam, golden, dev, base, oname, mode):
    cases.exp_log(pam, golden, dev, base, oname, mode)


def test_golden_pow(pam, golden, dev):
    cases.pow_(pam, golden, dev)


@pytest.mark.parametrize("tag,oname", [("ref21", "none"), ("ref20", "none"), ("rand", "none"), ("rand", "o1")])
@pytest.mark.parametrize("mode", ["exact", "approx"])
def test_golden_matmul(pam, golden, dev, tag, oname, mode):
    cases.matmul(pam, golden, dev, tag, oname, mode)


def test_golden_layouts_bmm_linear(pam, golden, dev):
    cases.matmul_layouts(pam, golden, dev)
    cases.bmm(pam, golden, dev)
    cases.linear_module(pam, golden, dev, exact_sums=False)


@pytest.mark.parametrize("oname,mode", cases.MODES)
def test_golden_reductions_layer_norm(pam, golden, dev, oname, mode):
    cases.reductions(pam, golden, dev, oname, mode, exact_sums=False)
    cases.layer_norm(pam, golden, dev, oname, mode, exact_sums=False)


def test_golden_cross_entropy_and_adam(pam, golden, dev):
    from pam_b200 import factories, optim
    cases.cross_entropy(pam, factories, golden, dev, exact_sums=False)
    cases.adam(optim, golden, dev)


def test_reference_known_answers_on_gpu(pam, dev):
    # pam/test_pam.py:13-29 and :36-43, run as the reference runs them (allclose / non-finite)
    abc = torch.tensor([
        [1.0, 1.0, 1.0], [1.2345, 1.0, 1.2345], [1.2345, 32.0, 32.0 * 1.2345],
        [-1.2345, 32.0, -32.0 * 1.2345], [1.2345, -32.0, -32.0 * 1.2345], [-1.2345, -32.0, 32.0 * 1.2345],
        [1.0, 0.0, 0.0], [0.0, -1.0, -0.0], [1.5, 1.5, 2.0], [1.3, -1.3, -1.6],
        [4.5, 3.0, 8 * (1 + (4.5 - 4) / 4 + (3.0 - 2) / 2)], [-6.0, 3.0, -16.0],
        [-3.5, -3.5, 8 * (1 + (3.5 - 2) / 2 + (3.5 - 2) / 2 - 1)], [1e-30, 1e-30, 0.0], [1e-30, -1e-30, -0.0],
    ], device=dev)
    for method in (pam.cuda_bindings.pam, pam.native.pam):
        assert torch.allclose(abc[:, 2], method(abc[:, 0].contiguous(), abc[:, 1].contiguous()))
    ab = torch.tensor([[1e30, 1e30], [1e30, -1e30], [float("-inf"), 1e-20], [float("nan"), -1e-20],
                       [float("inf"), 0.0], [float("nan"), 0.0]], device=dev)
    assert (~pam.cuda_bindings.pam(ab[:, 0].contiguous(), ab[:, 1].contiguous()).isfinite()).all()


# ---- elementwise kernels against the oracle --------------------------------------------------------

def _wide(n, g, spread=40):
    return torch.randn(n, generator=g) * torch.exp2(torch.randint(-spread, spread, (n,), generator=g).float())


@pytest.mark.parametrize("n", [1, 3, 4, 5, 1023, 4096, 1_000_003])
@pytest.mark.parametrize("offset", [1.0, 1.0552])
def test_elementwise_sizes_and_specials(pam, K, dev, n, offset):
    g = torch.Generator().manual_seed(n)
    a, b, dc = inject(_wide(n, g), 0.05, g), inject(_wide(n, g), 0.05, g), _wide(n, g, 10)
    ck = pam.cuda_bindings.cuda_kernels
    ad, bd, dd = a.to(dev), b.to(dev), dc.to(dev)
    assert_bits_equal(ck.pam_fwd(ad, bd, offset), K.pam_fwd(a, b, offset), "pam")
    assert_bits_equal(ck.pad_fwd(ad, bd, offset), K.pad_fwd(a, b, offset), "pad")
    assert_bits_equal(ck.pam_bwd(ad, bd, dd, offset), K.pam_bwd(a, b, dc, offset), "pam_bwd")
    assert_bits_equal(ck.pad_bwd(ad, bd, dd, offset), K.pad_bwd(a, b, dc, offset), "pad_bwd")


def test_elementwise_raw_bit_patterns(pam, K, dev):
    g = torch.Generator().manual_seed(11)
    n = 2_000_000
    a, b, dc = (torch.randint(-2**31, 2**31 - 1, (n,), generator=g, dtype=torch.int64).to(torch.int32)
                .view(torch.float32) for _ in range(3))
    ck = pam.cuda_bindings.cuda_kernels
    ad, bd, dd = a.to(dev), b.to(dev), dc.to(dev)
    assert_bits_equal(ck.pam_fwd(ad, bd, 1.0), K.pam_fwd(a, b, 1.0))
    assert_bits_equal(ck.pad_fwd(ad, bd, 1.0), K.pad_fwd(a, b, 1.0))
    assert_bits_equal(ck.pam_bwd(ad, bd, dd, 0.97), K.pam_bwd(a, b, dc, 0.97))
    assert_bits_equal(ck.pad_bwd(ad, bd, dd, 0.97), K.pad_bwd(a, b, dc, 0.97))


def test_elementwise_misaligned_views_and_guard_bands(pam, K, dev):
    """Operands that start 4 bytes off a 16-byte boundary take the scalar path; the kernel must
    not write outside its output (checked with canaries around a hand-placed output)."""
    from pam_b200 import _lib
    g = torch.Generator().manual_seed(5)
    n = 10_001
    a, b = _wide(n + 1, g), _wide(n + 1, g)
    ad, bd = a.to(dev)[1:], b.to(dev)[1:]
    assert ad.data_ptr() % 16 == 4
    want = K.pam_fwd(a[1:], b[1:], 1.0)
    assert_bits_equal(pam.cuda_bindings.cuda_kernels.pam_fwd(ad, bd, 1.0), want)
    for lead in (64, 65):                     # aligned and misaligned output start
        buf = torch.full((lead + n + 64,), 12345.0, device=dev)
        out = buf[lead:lead + n]
        h = _lib.lib()
        _lib.check(h.pamk_pam_fwd(ad.data_ptr(), 0, 0.0, bd.data_ptr(), 0, 0.0, out.data_ptr(), n, 0, 1.0,
                                  torch.cuda.current_stream().cuda_stream), "pam_fwd")
        assert_bits_equal(out, want)
        assert bool((buf[:lead] == 12345.0).all()) and bool((buf[lead + n:] == 12345.0).all())


@pytest.mark.parametrize("inner", [1, 4, 7, 192, 1000])
def test_elementwise_broadcast_kinds(pam, K, dev, inner):
    g = torch.Generator().manual_seed(inner)
    rows = 37
    m, row, col = _wide(rows * inner, g).view(rows, inner), _wide(inner, g), _wide(rows, g).view(rows, 1)
    ck = pam.cuda_bindings.cuda_kernels
    md, rd, cd = m.to(dev), row.to(dev), col.to(dev)
    for other, od in ((row, rd), (col, cd), (col[3, 0], cd[3, 0]), (0.3, 0.3)):
        full = other.expand(rows, inner).contiguous() if isinstance(other, torch.Tensor) else torch.full((rows, inner), other)
        assert_bits_equal(ck.pam_fwd(md, od, 1.0), K.pam_fwd(m, full, 1.0), "pam rhs")
        assert_bits_equal(ck.pad_fwd(od, md, 1.0), K.pad_fwd(full, m, 1.0), "pad lhs")
        assert_bits_equal(ck.pam_bwd(md, od, md, 1.0), K.pam_bwd(m, full, m, 1.0), "pam_bwd")
        assert_bits_equal(ck.pad_bwd(md, od, od, 1.0), K.pad_bwd(m, full, full, 1.0), "pad_bwd")
    # an expanded (stride-0) view is described, not materialised, and gives the same bits
    assert_bits_equal(ck.pam_fwd(md, cd.expand(rows, inner), 1.0), K.pam_fwd(m, col.expand(rows, inner).contiguous(), 1.0))


def _near_pow2_below(x):
    """Inputs within 2 ulp below a power of two: floor(log2f(x)) legitimately depends on the
    libm in use (device vs host), and with it the piecewise-affine segment."""
    bits = x.view(torch.int32) & 0x7FFFFFFF
    return (bits & 0x007FFFFF) >= 0x007FFFFE


@pytest.mark.parametrize("base", [2.0, math.e, 10.0, 0.5])
@pytest.mark.parametrize("offset", [1.0, 1.0552])
def test_exp_log_against_oracle(pam, K, dev, base, offset):
    g = torch.Generator().manual_seed(21)
    n = 500_000
    x = torch.cat([torch.randn(n, generator=g) * 30, _wide(n, g, 60), inject(torch.randn(1000, generator=g), 0.5, g,
                  extra=(float("inf"), float("-inf"), float("nan"), 127.5, -126.5, -149.5, 128.0)),
                   torch.arange(-170, 140).float(), torch.arange(-170, 140).float() - 2.0 ** -18,
                   # results that are denormal, zero or infinite, and exponents far outside fp32's range
                   torch.arange(-320, 320).float() + 0.37, torch.arange(-160, -120).float() + 0.999999,
                   torch.tensor([-252.0, -252.5, -253.0, -251.5, 253.5, 254.0, 254.5, 255.0, 1e30, -1e30, 3e38, -3e38,
                                 -149.0, -150.0, -150.5, -151.0, 127.999, 128.5, -126.0, -127.0])])
    dy = _wide(x.numel(), g, 30)
    ck = pam.cuda_bindings.cuda_kernels
    xd, dd = x.to(dev), dy.to(dev)
    assert_bits_equal(ck.pa_exp_fwd(xd, base, offset), K.pa_exp_fwd(x, base, offset), "exp")
    assert_bits_equal(ck.pa_exp_bwd(xd, dd, base, offset), K.pa_exp_bwd(x, dy, base, offset), "exp_bwd")
    # log: every binade, both ends of each, plus random magnitudes
    e = torch.arange(0, 255, dtype=torch.int32)
    m = torch.tensor([0, 1, 2, 0x400000, 0x7FFFFD, 0x7FFFFE, 0x7FFFFF], dtype=torch.int32)
    grid = ((e[:, None] << 23) | m[None, :]).reshape(-1).view(torch.float32)
    xl = torch.cat([grid, _wide(n, g, 60).abs(), torch.tensor([0.0, -1.0, float("inf"), float("nan")])])
    dl = _wide(xl.numel(), g, 30)
    got, want = ck.pa_log_fwd(xl.to(dev), base, offset).cpu(), K.pa_log_fwd(xl, base, offset)
    gotb, wantb = ck.pa_log_bwd(xl.to(dev), dl.to(dev), base, offset).cpu(), K.pa_log_bwd(xl, dl, base, offset)
    sure = ~_near_pow2_below(xl)
    assert_bits_equal(got[sure], want[sure], "log")
    assert_bits_equal(gotb[sure], wantb[sure], "log_bwd")
    # just below a power of two either segment is a legitimate answer; they meet there, so the
    # values agree closely even when the bits do not
    edge = ~sure & want.isfinite()
    assert_close_nan(got[edge], want[edge], 1e-5, 1e-6, "log at binade edge")


# ---- matrix products against the oracle -------------------------------------------------------------

SHAPES = [(1, 1, 1), (5, 3, 4), (33, 31, 1), (17, 19, 23), (128, 128, 16), (129, 130, 17), (257, 64, 100),
          (64, 300, 48), (200, 192, 192)]


def _layouts(A, B):
    yield "rm x rm", A, B
    yield "rm x cm", A, B.T.contiguous().T
    yield "cm x rm", A.T.contiguous().T, B
    yield "cm x cm", A.T.contiguous().T, B.T.contiguous().T


@pytest.mark.parametrize("M,N,Kdim", SHAPES)
def test_matmul_shapes_layouts_bit_exact(pam, K, dev, tile, M, N, Kdim):
    g = torch.Generator().manual_seed(M * 1000 + N)
    A, B = torch.randn(M, Kdim, generator=g), torch.randn(Kdim, N, generator=g) * 0.02
    want = K.pam_matmul_fwd(A, B)
    std = K.standard_matmul(A, B)
    ck = pam.cuda_bindings.cuda_kernels
    for name, a, b in _layouts(A.to(dev), B.to(dev)):
        assert_bits_equal(ck.pam_matmul_fwd(a, b, True, True, 1.0), want, f"pam {name}")
        assert_bits_equal(ck.standard_matmul(a, b), std, f"standard {name}")
    D = torch.randn(M, N, generator=g)
    for delta_l in (True, False):
        wantb = K.pam_matmul_bwd(A, B, D, True, True, delta_l, 1.0552)
        for name, a, b in _layouts(A.to(dev), B.to(dev)):
            assert_bits_equal(ck.pam_matmul_bwd(a, b, D.to(dev), True, True, delta_l, 1.0552), wantb,
                              f"bwd {name} delta_l={delta_l}")


@pytest.mark.parametrize("frac", [0.01, 0.3])
@pytest.mark.parametrize("offset", [1.0, 1.0552])
def test_matmul_special_values_bit_exact(pam, K, dev, tile, frac, offset):
    """Zeros, denormals, +-1e30 / +-1e-30, inf and NaN in the operands: the hoisted range rule must
    reproduce flush-to-+0, NaN-on-overflow and raw-bit denormal products exactly."""
    g = torch.Generator().manual_seed(int(frac * 100))
    A = inject(torch.randn(150, 260, generator=g), frac, g)
    B = inject(torch.randn(260, 140, generator=g), frac, g)
    A[7, 100] = float("inf")
    B[33, 5] = float("nan")
    A[100:110] = 0.0                    # an all-zero row block (padding-like)
    want = K.pam_matmul_fwd(A, B, True, True, offset)
    assert want.isnan().any() and (~want.isnan()).any()
    for name, a, b in _layouts(A.to(dev), B.to(dev)):
        assert_bits_equal(pam.cuda_bindings.cuda_kernels.pam_matmul_fwd(a, b, True, True, offset), want, name)


def test_matmul_tiny_and_huge_magnitudes(pam, K, dev, tile):
    """Operands whose exponent ranges make the per-slab classification take each branch: all
    products far in range, products straddling the 1e-37 flush threshold, and straddling 1e37."""
    g = torch.Generator().manual_seed(3)
    for scale_a, scale_b in ((1.0, 1.0), (1e-19, 1e-19), (1e-18, 3e-20), (1e18, 1e19), (3e18, 3e18), (1e-30, 1e30)):
        A = torch.randn(96, 80, generator=g) * scale_a
        B = torch.randn(80, 72, generator=g) * scale_b
        want = K.pam_matmul_fwd(A, B)
        got = pam.cuda_bindings.cuda_kernels.pam_matmul_fwd(A.to(dev), B.to(dev), True, True, 1.0)
        assert_bits_equal(got, want, f"scales {scale_a} x {scale_b}")


def test_bmm_bit_exact_and_guard_bands(pam, K, dev, tile):
    from pam_b200 import _lib
    g = torch.Generator().manual_seed(8)
    A, B = torch.randn(11, 13, 15, generator=g), torch.randn(11, 15, 19, generator=g)
    want = K.pam_bmm_fwd(A, B)
    ck = pam.cuda_bindings.cuda_kernels
    assert_bits_equal(ck.pam_bmm_fwd(A.to(dev), B.to(dev), True, True, 1.0), want)
    # batch-transposed views (attention's k.transpose(-1, -2))
    Bt = B.transpose(1, 2).contiguous().transpose(1, 2)
    assert_bits_equal(ck.pam_bmm_fwd(A.to(dev), Bt.to(dev), True, True, 1.0), want)
    D = torch.randn(11, 13, 19, generator=g)
    assert_bits_equal(ck.pam_bmm_bwd(A.to(dev), B.to(dev), D.to(dev), True, True, True, 1.0),
                      K.pam_bmm_bwd(A, B, D, True, True, True, 1.0))
    # output written in place between canaries
    count = 11 * 13 * 19
    buf = torch.full((256 + count + 256,), -7.0, device=dev)
    out = buf[256:256 + count]
    Ad, Bd = A.to(dev), B.to(dev)
    _lib.check(_lib.lib().pamk_matmul(0, Ad.data_ptr(), Bd.data_ptr(), out.data_ptr(), 11, 13, 19, 15,
                                      *Ad.stride(), *Bd.stride(), 1.0, 1, None, 0,
                                      torch.cuda.current_stream().cuda_stream), "matmul")
    assert_bits_equal(out.view(11, 13, 19), want)
    assert bool((buf[:256] == -7.0).all()) and bool((buf[256 + count:] == -7.0).all())


def _sum_abs_products(K, A, B):
    return K.pam_matmul_fwd(A.abs(), B.abs()).double()


@pytest.mark.parametrize("split", [2, 4, 5, 8, 16, 24])
def test_matmul_split_k_within_tolerance(pam, K, dev, tile, split):
    """Split-K adds the same bit-exact products in a different association.  Bound for any
    order: |C - S| <= 2 * K * 2^-24 * sum|p_k|  (S the exact sum of the products)."""
    from pam_b200 import cuda_bindings as cb
    g = torch.Generator().manual_seed(split)
    M, N, Kdim = 100, 70, 1000
    A, B = torch.randn(M, Kdim, generator=g), torch.randn(Kdim, N, generator=g)
    seq = K.pam_matmul_fwd(A, B)
    got = cb._matmul(0, A.to(dev), B.to(dev), 1.0, 2, split_k=split).cpu()
    bound = 2 * Kdim * 2.0 ** -24 * _sum_abs_products(K, A, B)
    err = (got.double() - seq.double()).abs()
    assert bool((err <= 2 * bound).all())          # both sums are within `bound` of S
    assert float((err / (2.0 ** -24 * _sum_abs_products(K, A, B))).max()) < 4 * math.sqrt(Kdim)
    # and it is deterministic
    again = cb._matmul(0, A.to(dev), B.to(dev), 1.0, 2, split_k=split).cpu()
    assert torch.equal(got, again)


@pytest.mark.parametrize("split", [2, 7, 32])
@pytest.mark.parametrize("delta_l", [True, False])
def test_exact_gradient_split_k_within_tolerance(pam, K, dev, tile, split, delta_l):
    """The exact-gradient product with K split (weight gradients contract over the token count):
    the same bit-exact terms delta * slope, added in a different association."""
    from pam_b200 import cuda_bindings as cb
    g = torch.Generator().manual_seed(split + 10 * delta_l)
    M, N, Kdim = 70, 90, 2000
    L, R, D = torch.randn(M, Kdim, generator=g), torch.randn(Kdim, N, generator=g), torch.randn(M, N, generator=g)
    seq = K.pam_matmul_bwd(L, R, D, True, True, delta_l, 1.0)
    got = cb._matmul_bwd(L.to(dev), R.to(dev), D.to(dev), delta_l, 1.0, 2, split_k=split).cpu()
    terms = K.pam_matmul_bwd(L.abs(), R.abs(), D.abs(), True, True, delta_l, 1.0).double()     # sum of |delta * slope|
    err = (got.double() - seq.double()).abs()
    assert bool((err <= 4 * Kdim * 2.0 ** -24 * terms).all())
    assert float((err / (2.0 ** -24 * terms)).max()) < 4 * math.sqrt(Kdim)
    assert torch.equal(got, cb._matmul_bwd(L.to(dev), R.to(dev), D.to(dev), delta_l, 1.0, 2, split_k=split).cpu())
    # split_k = 1 is the reference's order
    assert_bits_equal(cb._matmul_bwd(L.to(dev), R.to(dev), D.to(dev), delta_l, 1.0, 2, split_k=1), seq, "unsplit")


def test_config1_matmul_forward_and_approx_backward(pam, K, dev):
    """BASELINE config 1: A[512x1024] . B[1024x512], N(0,1), forward plus approx_bwd backward with
    N(0,1) grad_out; per-product results on a sampled block and all three products bit-exact."""
    g = torch.Generator().manual_seed(1)
    A, B, G = torch.randn(512, 1024, generator=g), torch.randn(1024, 512, generator=g), torch.randn(512, 512, generator=g)
    Ad, Bd = A.to(dev).requires_grad_(), B.to(dev).requires_grad_()
    C = pam.matmul(Ad, Bd, approx_bwd=True)
    C.backward(G.to(dev))
    assert_bits_equal(C, K.pam_matmul_fwd(A, B), "C")
    assert_bits_equal(Ad.grad, K.pam_matmul_fwd(G, B.T), "dA")
    assert_bits_equal(Bd.grad, K.pam_matmul_fwd(A.T, G), "dB")
    # per-product check on rows 0..63 x all K x cols 0..63 through the elementwise kernel
    prod = pam.mul(A[:64, :, None].to(dev), B[None, :, :64].to(dev))
    want = K.pam_fwd(A[:64, :, None].expand(64, 1024, 64).contiguous(), B[None, :, :64].expand(64, 1024, 64).contiguous(), 1.0)
    assert_bits_equal(prod, want, "per-product")


def test_deit_linear_set_bit_exact_on_row_sample(pam, K, dev, tile):
    """BASELINE config 2 shapes (M = 12608 tokens, 192->576, 192->192, 192->768, 768->192,
    trunc-normal(0.02) weights): full-size products on the GPU, checked bit for bit on a sample of
    rows against the oracle, forward and both approx_bwd gradients."""
    g = torch.Generator().manual_seed(2)
    M = 12608
    rows = torch.randperm(M, generator=g)[:96]
    for k_in, n_out in ((192, 576), (192, 192), (192, 768), (768, 192)):
        X = torch.randn(M, k_in, generator=g)
        W = torch.nn.init.trunc_normal_(torch.empty(n_out, k_in), std=0.02, generator=g)
        G = torch.randn(M, n_out, generator=g)
        Xd, Wd = X.to(dev).requires_grad_(), W.to(dev).requires_grad_()
        Y = pam.linear(Xd, Wd, approx_bwd=True)
        Y.backward(G.to(dev))
        assert_bits_equal(Y[rows.to(dev)], K.pam_matmul_fwd(X[rows], W.T), f"Y {k_in}->{n_out}")
        assert_bits_equal(Xd.grad[rows.to(dev)], K.pam_matmul_fwd(G[rows], W), f"dX {k_in}->{n_out}")
        cols = torch.arange(0, k_in, 7)
        assert_bits_equal(Wd.grad[:, cols.to(dev)], K.pam_matmul_fwd(G.T, X[:, cols]), f"dW {k_in}->{n_out}")


def test_square_gemm_4096_with_specials_sampled(pam, K, dev):
    """Scaling-sweep configuration at 4096^3 with 1% injected special values: a 48x48 block of the
    output (full K) must match the oracle bit for bit, and permuting the rows of A must permute the
    rows of C (a size-independent property of the per-output summation)."""
    g = torch.Generator().manual_seed(4)
    n = 4096
    A = inject(torch.randn(n, n, generator=g), 0.01, g)
    B = inject(torch.randn(n, n, generator=g), 0.01, g)
    Ad, Bd = A.to(dev), B.to(dev)
    ck = pam.cuda_bindings.cuda_kernels
    C = ck.pam_matmul_fwd(Ad, Bd, True, True, 1.0)
    r = torch.randperm(n, generator=g)[:48]
    c = torch.randperm(n, generator=g)[:48]
    assert_bits_equal(C[r.to(dev)][:, c.to(dev)], K.pam_matmul_fwd(A[r], B[:, c]), "sampled block")
    perm = torch.randperm(n, generator=g).to(dev)
    Cp = ck.pam_matmul_fwd(Ad[perm], Bd, True, True, 1.0)
    assert bool(bits_equal(Cp, C[perm]).all())


# ---- the reference's own test recipes, run as the reference runs them ---------------------------------

def test_reference_recipe_conv_and_bmm_power_of_two_equivalence(pam, dev):
    """pam/test_pam.py:151-216: with power-of-two weights and short-mantissa inputs PAM equals true
    multiplication, so conv2d / grouped conv / bmm must match torch's outputs and both gradients
    (odd sizes exercise the tile edges)."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    g = torch.Generator().manual_seed(17)
    close = lambda a, b: torch.allclose(a, b, rtol=1e-5, atol=1e-3)

    X = (torch.randint(-1024, 1024, (11, 13, 15, 17), generator=g) / 64.0).to(dev).requires_grad_()
    W = (2.0 ** torch.randint(-8, 8, (19, 13, 3, 5), generator=g)).to(dev).requires_grad_()
    X2, W2 = X.detach().clone().requires_grad_(), W.detach().clone().requires_grad_()
    Y = pam.conv2d(X, W, approx_bwd=True)
    Y.sum().backward()
    Y2 = torch.nn.functional.conv2d(X2, W2)
    Y2.sum().backward()
    assert close(Y, Y2) and close(X.grad, X2.grad) and close(W.grad, W2.grad)

    for G in (1, 8):
        X = (torch.randint(-8, 9, (11, 16, 15, 17), generator=g) / 4.0).to(dev).requires_grad_()
        W = (2.0 ** torch.randint(-2, 3, (128, 16 // G, 3, 5), generator=g)).to(dev).requires_grad_()
        X2, W2 = X.detach().clone().requires_grad_(), W.detach().clone().requires_grad_()
        Y = pam.conv2d_group(X, W, groups=G, approx_bwd=True)
        Y.sum().backward()
        Y2 = torch.nn.functional.conv2d(X2, W2, groups=G)
        Y2.sum().backward()
        assert close(Y, Y2) and close(X.grad, X2.grad) and close(W.grad, W2.grad)

    X = (torch.randint(-128, 128, (11, 13, 15), generator=g) / 64.0).to(dev).requires_grad_()
    W = (2.0 ** torch.randint(-8, 8, (11, 15, 19), generator=g)).to(dev).requires_grad_()
    X2, W2 = X.detach().clone().requires_grad_(), W.detach().clone().requires_grad_()
    Y = pam.bmm(X, W, approx_bwd=True)
    Y.sum().backward()
    Y2 = torch.bmm(X2, W2)
    Y2.sum().backward()
    assert close(Y, Y2) and close(X.grad, X2.grad) and close(W.grad, W2.grad)


def test_reference_recipe_exact_gradient_and_bmm_bwd(pam, oracle, dev):
    """pam/test_pam.py:48-73 (exact backward of the elementwise product on exponents in [-30, 30))
    and :219-239 (batched product with the exact backward), against the oracle."""
    g = torch.Generator().manual_seed(18)
    n = 128
    A = (2.0 ** torch.randint(-30, 30, (n,), generator=g)) * (1 + torch.rand(n, generator=g))
    B = (2.0 ** torch.randint(-30, 30, (n,), generator=g)) * (1 + torch.rand(n, generator=g))
    dC = torch.arange(n).float()
    A1, B1 = A.to(dev).requires_grad_(), B.to(dev).requires_grad_()
    pam.cuda_bindings.pam(A1, B1).backward(dC.to(dev))
    A2, B2 = A.clone().requires_grad_(), B.clone().requires_grad_()
    oracle.mul(A2, B2).backward(dC)
    assert_bits_equal(A1.grad, A2.grad)
    assert_bits_equal(B1.grad, B2.grad)

    X = torch.randint(-1024, 1024, (11, 13, 15), generator=g) / 32.0
    W = torch.randint(-1024, 1024, (11, 15, 19), generator=g) / 32.0
    X1, W1 = X.to(dev).requires_grad_(), W.to(dev).requires_grad_()
    Y1 = pam.bmm(X1, W1, approx_bwd=False)
    Y1.sum().backward()
    X2, W2 = X.clone().requires_grad_(), W.clone().requires_grad_()
    Y2 = oracle.bmm(X2, W2, approx_bwd=False)
    Y2.sum().backward()
    assert_bits_equal(Y1, Y2)
    assert_bits_equal(X1.grad, X2.grad)
    assert_bits_equal(W1.grad, W2.grad)


def test_empty_and_degenerate_inputs(pam, dev):
    e = torch.empty(0, device=dev)
    assert pam.mul(e, e).shape == (0,) and pam.div(e, 2.0).shape == (0,) and pam.exp2(e).shape == (0,)
    assert pam.matmul(torch.empty(0, 5, device=dev), torch.ones(5, 3, device=dev)).shape == (0, 3)
    z = pam.matmul(torch.ones(4, 0, device=dev), torch.ones(0, 3, device=dev))          # K = 0: all sums are +0
    assert z.shape == (4, 3) and bool((z == 0).all())
    assert pam.bmm(torch.empty(0, 2, 3, device=dev), torch.empty(0, 3, 4, device=dev)).shape == (0, 2, 4)
    ln = pam.LayerNorm(8).to(dev)
    assert ln(torch.empty(0, 8, device=dev)).shape == (0, 8)
    assert pam.softmax(torch.empty(0, 7, device=dev), dim=-1).shape == (0, 7)
    one = pam.softmax(torch.tensor([[3.0]], device=dev), dim=-1)                          # single-entry rows
    assert one.item() == 1.0
    # non-contiguous inputs: a strided view and a transposed matrix give the contiguous copy's result
    x = torch.randn(16, 32, device=dev)
    assert torch.equal(pam.mul(x[:, ::2], 1.5), pam.mul(x[:, ::2].contiguous(), 1.5))
    assert torch.equal(pam.softmax(x.T, dim=-1), pam.softmax(x.T.contiguous(), dim=-1))
    assert torch.equal(pam.layer_norm(x.T, (16,)), pam.layer_norm(x.T.contiguous(), (16,)))


# ---- fused layer normalisation ---------------------------------------------------------------------

def _ln_vec(width):
    """Columns per register chunk of the pam_ln layout the library picks for aligned rows."""
    if width % 4 == 0 and width <= 128:
        return 4
    if width % 2 == 0 and width <= 192:
        return 2
    return 4 if width % 4 == 0 else 1


def _ln_rows_per_warp(width, approx=False):
    """Rows a warp of the backward kernel handles per pass: four for layouts of up to 8 register
    slots per lane, two up to 16, else one (pam_b200/csrc/layer_norm.cu rows_per_warp_bwd); the
    approximate backward, which works from the row scalars the forward pass saved, takes two rows
    for layouts of up to 8 slots and one otherwise."""
    vec = _ln_vec(width)
    if vec == 4:
        slots = next(s for cap, s in ((128, 4), (256, 8), (512, 16), (768, 24), (1024, 32)) if width <= cap)
    elif vec == 2:
        slots = 6
    else:
        slots = 8 if width <= 256 else 32
    if approx:
        return 2 if slots <= 8 else 1
    return 4 if slots <= 8 else (2 if slots <= 16 else 1)


def _ln_case(pam, dev, rows, width, affine, approx, offset, seed):
    import ln_emulation as E
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, width, generator=g) * 2 + 0.3
    gy = torch.randn(rows, width, generator=g)
    w = (torch.randn(width, generator=g).abs() + 0.5) if affine else None
    b = torch.randn(width, generator=g) if affine else None
    xd = x.to(dev).requires_grad_()
    wd = w.to(dev).requires_grad_() if affine else None
    bd = b.to(dev).requires_grad_() if affine else None
    y = pam.layer_norm(xd, (width,), wd, bd, 1e-5, offset=offset, approx_bwd=approx)
    y.backward(gy.to(dev))
    vec = _ln_vec(width)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    grid = min((rows + 3) // 4, sms * 12)                    # CTAs of the backward kernel
    chain = E.Chain(offset, E.kernel_rowsum(vec), E.kernel_colsum(rows, grid, rows_per_warp=_ln_rows_per_warp(width, approx)))
    want = chain.run(x, w, b, gy, 1e-5, approx)
    got = (y, xd.grad, wd.grad if affine else None, bd.grad if affine else None)
    return got, want


@pytest.mark.parametrize("width", [1, 2, 5, 48, 130, 192, 200, 512, 768, 1000, 1024])
@pytest.mark.parametrize("approx", [True, False])
def test_fused_layer_norm_bit_exact_against_replayed_chain(pam, dev, width, approx):
    """The kernel against the CPU replay of its own chain in its own summation order: every output
    and gradient bit for bit.  (The same chain summed with torch.sum is checked against the
    reference's fixtures in test_oracle_golden.py.)"""
    for affine, offset, rows in ((True, None, 37), (False, 1.0552, 5), (True, None, 7500)):
        if rows > 100 and width not in (48, 192):
            continue                                          # the long case walks several rows per warp
        got, want = _ln_case(pam, dev, rows, width, affine, approx, offset, width)
        for name, a, b in zip(("y", "dx", "dw", "db"), got, want):
            if b is not None:
                assert_bits_equal(a.reshape(b.shape), b, f"ln {name} width={width} affine={affine}")


@pytest.mark.parametrize("approx", [True, False])
def test_fused_layer_norm_matches_unfused_route(pam, dev, approx):
    """Fused kernel vs the one-kernel-per-primitive composition on the GPU (torch.sum reductions):
    same values up to the association of the row sums."""
    from pam_b200 import fused
    g = torch.Generator().manual_seed(9)
    x = torch.randn(4, 197, 192, generator=g).to(dev)
    gy = torch.randn(4, 197, 192, generator=g).to(dev)
    ln = pam.LayerNorm(192, eps=1e-6, approx_bwd=approx).to(dev)
    outs = []
    for flag in (True, False):
        fused.enabled = flag
        try:
            xi = x.clone().requires_grad_()
            ln.zero_grad()
            y = ln(xi)
            y.backward(gy)
            outs.append((y.detach(), xi.grad, ln.weight.grad.clone(), ln.bias.grad.clone()))
        finally:
            fused.enabled = True
    for name, a, b in zip(("y", "dx", "dw", "db"), *outs):
        if approx or name in ("y", "db"):
            assert_close_nan(a, b, 2e-4, 2e-4 * float(b.abs().max()), f"ln {name}")
        else:
            # exact slopes are step functions of the centred values: a last-bit difference in a row
            # mean can move an element across a step, so compare the bulk of the distribution
            close = torch.isclose(a, b, rtol=2e-3, atol=2e-3 * float(b.abs().max()))
            assert float(close.float().mean()) > 0.98, f"ln {name}"


def test_layer_norm_config2_rows(pam, dev):
    """BASELINE config 2: pam_ln over the 192-wide rows of X[12608 x 192], gamma = 1, beta = 0,
    approx_bwd: full size on the GPU against the replayed chain on a sample of rows."""
    import ln_emulation as E
    g = torch.Generator().manual_seed(12)
    x, gy = torch.randn(12608, 192, generator=g), torch.randn(12608, 192, generator=g)
    ln = pam.LayerNorm(192, eps=1e-6, approx_bwd=True).to(dev)
    xd = x.to(dev).requires_grad_()
    y = ln(xd)
    y.backward(gy.to(dev))
    rows = torch.randperm(12608, generator=g)[:64]
    chain = E.Chain(None, E.kernel_rowsum(_ln_vec(192)), E.torch_colsum)
    wy, wdx, _, _ = chain.run(x[rows], torch.ones(192), torch.zeros(192), gy[rows], 1e-6, True)
    assert_bits_equal(y[rows.to(dev)], wy, "y")
    assert_bits_equal(xd.grad[rows.to(dev)], wdx, "dx")
    assert_close_nan(ln.bias.grad, gy.sum(0), 1e-4, 1e-3, "db")


# ---- fused softmax / logsumexp -----------------------------------------------------------------------

def _row_order(length):
    """(vec, warps) of the row kernel the library picks for contiguous, 16-byte aligned rows."""
    vec = 4 if length % 4 == 0 else 1
    return vec, (1 if length <= 1024 else 8)


@pytest.mark.parametrize("length", [1, 5, 32, 60, 64, 100, 128, 130, 197, 200, 224, 225, 256, 300, 512, 516, 768, 772, 1000, 1024, 1028, 4096, 10000])
@pytest.mark.parametrize("approx", [True, False])
def test_fused_softmax_logsumexp_bit_exact_against_replayed_chain(pam, dev, length, approx):
    import ln_emulation as E
    g = torch.Generator().manual_seed(length)
    rows = 9
    for offset in (None, 1.0552):
        x = torch.randn(rows, length, generator=g) * 3
        gy = torch.randn(rows, length, generator=g)
        chain = E.Chain(offset, E.kernel_rowsum(*_row_order(length)), E.torch_colsum)
        # softmax with attention-style masking (-inf) in some rows
        xm = x.clone()
        if length > 2:
            xm[::2, -(length // 3 + 1):] = float("-inf")
        xd = xm.to(dev).requires_grad_()
        y = pam.softmax(xd, dim=-1, offset=offset, approx_bwd=approx)
        y.backward(gy.to(dev))
        wy, wdx = chain.softmax(xm, gy, approx)
        assert_bits_equal(y, wy, f"softmax len={length}")
        assert_bits_equal(xd.grad, wdx, f"softmax dx len={length}")
        # logsumexp and log_softmax (finite inputs)
        xd = x.to(dev).requires_grad_()
        z = pam.logsumexp(xd, dim=-1, offset=offset, approx_bwd=approx)
        z.backward(gy[:, 0].to(dev))
        wz, wdz = chain.logsumexp(x, gy[:, 0], approx)
        assert_bits_equal(z, wz, f"logsumexp len={length}")
        assert_bits_equal(xd.grad, wdz, f"logsumexp dx len={length}")


def test_fused_softmax_shift_is_global_and_nan_is_sticky(pam, dev):
    import ln_emulation as E
    g = torch.Generator().manual_seed(5)
    x = torch.randn(3000, 64, generator=g)
    x[2999, 63] = 40.0                       # the maximum sits in the last row: every row's shift moves
    y = pam.softmax(x.to(dev), dim=-1)
    wy, _ = E.Chain(None, E.kernel_rowsum(4, 1), E.torch_colsum).softmax(x, torch.zeros_like(x), True)
    assert_bits_equal(y, wy)
    # a fully masked row is NaN (0 / 0 through PAM division), the others are untouched
    xm = x.clone()
    xm[7] = float("-inf")
    ym = pam.softmax(xm.to(dev), dim=-1).cpu()
    assert ym[7].isnan().all() and torch.equal(ym[8], wy[8])
    # +inf or NaN anywhere poisons the whole-tensor shift, as with torch.max in the reference
    xn = x.clone()
    xn[5, 5] = float("nan")
    assert pam.softmax(xn.to(dev), dim=-1).isnan().all()


def test_fused_softmax_matches_unfused_route(pam, dev):
    from pam_b200 import fused
    g = torch.Generator().manual_seed(6)
    x = (torch.randn(12, 197, 197, generator=g) * 2).to(dev)        # DeiT attention scores, one layer / 4 images
    gy = torch.randn(12, 197, 197, generator=g).to(dev)
    outs = []
    for flag in (True, False):
        fused.enabled = flag
        try:
            xi = x.clone().requires_grad_()
            y = pam.softmax(xi, dim=-1, approx_bwd=True)
            y.backward(gy)
            z = pam.log_softmax(xi, dim=-1, approx_bwd=True)
            outs.append((y.detach(), xi.grad.clone(), z.detach()))
        finally:
            fused.enabled = True
    for name, a, b in zip(("y", "dx", "log_softmax"), *outs):
        assert_close_nan(a, b, 1e-4, 1e-5 * float(b.abs().max()) + 1e-7, name)


# ---- fused Adam ---------------------------------------------------------------------------------------

def test_fused_adam_many_tensors_bit_exact(pam, oracle, dev):
    """A table of tensors of awkward sizes (empty, one element, not a multiple of four, views that
    start off a 16-byte boundary, more tensors than one launch holds) through three steps, against
    the oracle's restatement of the reference rule; and the unfused op-dictionary route likewise."""
    from pam_b200 import optim
    g = torch.Generator().manual_seed(77)
    sizes = [0, 1, 3, 4, 5, 257, 1024, 4099] + [33 + 7 * i for i in range(30)]
    for cfg in ("pam", '{"type": "pam"}'):
        backing = [torch.randn(n + 1, generator=g) for n in sizes]
        params = [torch.nn.Parameter(b.to(dev)[1:] if i % 3 == 0 else b.to(dev)[:-1].clone()) for i, b in enumerate(backing)]
        host = [p.detach().cpu().clone() for p in params]
        ms = [torch.zeros_like(h) for h in host]
        vs = [torch.zeros_like(h) for h in host]
        opt = optim.Adam(params, lr=5e-4, betas=(0.9, 0.98), eps=1e-8, weight_decay=1e-4, opt_functional_cfg=cfg)
        for step in (1, 2, 3):
            grads = [torch.randn(h.shape, generator=g) * 0.1 for h in host]
            if step == 2:
                for gr in grads:
                    gr[::5] = 0.0
            for p, gr in zip(params, grads):
                p.grad = gr.to(dev)
            opt.step()
            for i in range(len(host)):
                host[i], ms[i], vs[i] = oracle.adam_step(host[i], grads[i], ms[i], vs[i], step=step, lr=5e-4,
                                                         betas=(0.9, 0.98), eps=1e-8, weight_decay=1e-4)
        for i, p in enumerate(params):
            assert_bits_equal(p.detach(), host[i], f"{cfg} p[{i}]")
            if sizes[i]:
                assert_bits_equal(opt.state[p]["exp_avg"], ms[i], f"{cfg} m[{i}]")
                assert_bits_equal(opt.state[p]["exp_avg_sq"], vs[i], f"{cfg} v[{i}]")


def test_abi_rejects_bad_arguments_on_gpu(pam, dev):
    from pam_b200 import _lib
    h = _lib.lib()
    x = torch.ones(64, device=dev)
    s = torch.cuda.current_stream().cuda_stream
    assert h.pamk_pam_fwd(x.data_ptr(), 9, 0.0, x.data_ptr(), 0, 0.0, x.data_ptr(), 64, 0, 1.0, s) == -1
    assert h.pamk_pam_fwd(x.data_ptr(), 2, 0.0, x.data_ptr(), 0, 0.0, x.data_ptr(), 64, 5, 1.0, s) == -1   # 64 % 5
    assert h.pamk_matmul(0, x.data_ptr(), x.data_ptr(), x.data_ptr(), 1, 4, 4, 4, 0, 8, 2, 0, 4, 1, 1.0, 1, None, 0, s) == -3
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        pam.mul(torch.ones(3), torch.ones(3))
    torch.cuda.synchronize()


# ---- linear layer with the bias in the product's epilogue ---------------------------------------------

@pytest.mark.parametrize("M,N,Kdim", [(1, 1, 1), (5, 3, 7), (64, 64, 16), (197, 130, 100), (300, 576, 192)])
@pytest.mark.parametrize("approx", [True, False])
def test_linear_bias_epilogue_bit_exact(pam, K, oracle, dev, tile, M, N, Kdim, approx):
    """y = X W^T + b with the add fused into the product: the same bits as the reference's product
    followed by a separate add; gradients of X and W as for the plain product; the bias gradient is
    a column sum (ordinary fp32 adds, compared with a float64 sum)."""
    g = torch.Generator().manual_seed(M * 31 + N)
    X, W, b = torch.randn(M, Kdim, generator=g), torch.randn(N, Kdim, generator=g) * 0.1, torch.randn(N, generator=g)
    G = torch.randn(M, N, generator=g)
    Xd, Wd, bd = (t.to(dev).requires_grad_() for t in (X, W, b))
    y = pam.linear(Xd, Wd, bd, approx_bwd=approx)
    y.backward(G.to(dev))
    assert_bits_equal(y, K.pam_matmul_fwd(X, W.T) + b, "y")
    if approx:
        assert_bits_equal(Xd.grad, K.pam_matmul_fwd(G, W), "dX")
        assert_bits_equal(Wd.grad, K.pam_matmul_fwd(G.T, X), "dW")
    else:
        assert_bits_equal(Xd.grad, K.pam_matmul_bwd(G, W, X, True, True, True, 1.0), "dX")
        assert_bits_equal(Wd.grad.T, K.pam_matmul_bwd(X.T, G, W.T, True, True, False, 1.0), "dW")
    want = G.double().sum(0)
    assert bool(((bd.grad.cpu().double() - want).abs() <= 1e-6 * G.abs().double().sum(0) + 1e-9).all())


def test_linear_bias_with_split_k_and_empty_k(pam, K, dev, tile):
    from pam_b200 import cuda_bindings as cb
    g = torch.Generator().manual_seed(77)
    X, W, b = torch.randn(40, 3000, generator=g), torch.randn(24, 3000, generator=g), torch.randn(24, generator=g)
    plain = cb._matmul(0, X.to(dev), W.T.to(dev), 1.0, 2, split_k=6)
    fused_ = cb._matmul(0, X.to(dev), W.T.to(dev), 1.0, 2, split_k=6, bias=b.to(dev))
    assert_bits_equal(fused_, plain.cpu() + b, "split-K: bias added after the partial sums")
    empty = cb._matmul(0, torch.empty(5, 0, device=dev), torch.empty(0, 24, device=dev), 1.0, 2, bias=b.to(dev))
    assert_bits_equal(empty, (torch.zeros(5, 24) + b), "K = 0: rows of bias")


@pytest.mark.parametrize("rows,cols", [(1, 1), (63, 5), (1000, 192), (12608, 768), (4096, 10000), (7, 130)])
def test_column_sum(pam, dev, rows, cols):
    from pam_b200 import cuda_bindings as cb
    g = torch.Generator().manual_seed(rows + cols)
    X = torch.randn(rows, cols, generator=g)
    got = cb._column_sum(X.to(dev))
    want = X.double().sum(0)
    bound = 2.0 ** -23 * math.sqrt(rows) * X.abs().double().sum(0) + 1e-12
    assert bool(((got.cpu().double() - want).abs() <= bound).all())
    assert torch.equal(got, cb._column_sum(X.to(dev)))
    # a view with a row stride is gathered first
    wide = torch.randn(rows, cols + 3, generator=g).to(dev)
    assert torch.equal(cb._column_sum(wide[:, :cols]), cb._column_sum(wide[:, :cols].contiguous()))


@pytest.mark.parametrize("length", [5, 64, 197, 512, 768, 1024, 4096, 10000])
@pytest.mark.parametrize("offset", [1.0, 1.0552])
def test_softmax_backward_from_saved_exponentials(pam, dev, length, offset):
    """pamk_softmax_fwd_save + pamk_softmax_bwd_saved against pamk_softmax_fwd + pamk_softmax_bwd(approx):
    the same bits, also where entries are masked (-inf), where exponentials underflow to zero, and where
    the incoming gradient is inf / NaN on such entries (a masked entry's gradient is 0 whatever arrives,
    an underflowed one's is NaN when inf arrives)."""
    from pam_b200 import _lib
    handle = _lib.lib()
    g = torch.Generator().manual_seed(length)
    rows = 37
    x = torch.randn(rows, length, generator=g) * 4
    x[::3, : max(1, length // 4)] = float("-inf")                 # masks
    x[1::5, -1] = -400.0                                          # exponentials that underflow to +0
    x[5] = float("-inf")                                          # a fully masked row
    dy = torch.randn(rows, length, generator=g)
    dy[0, 0] = float("inf")                                       # on a masked entry
    dy[1, -1] = float("inf")                                      # on an underflowed entry
    dy[2, length // 2] = float("nan")
    xd, dyd = x.to(dev), dy.to(dev)
    st = _lib.stream_ptr(dev)
    wsb = handle.pamk_softmax_workspace_bytes(rows, length)
    ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
    y0, y1, e, dx0, dx1, dx2 = (torch.empty_like(xd) for _ in range(6))
    with _lib.device_guard(dev):
        assert handle.pamk_softmax_fwd(xd.data_ptr(), y0.data_ptr(), rows, length, offset, ws.data_ptr(), wsb, st) == 0
        assert handle.pamk_softmax_fwd_save(xd.data_ptr(), y1.data_ptr(), e.data_ptr(), rows, length, offset, ws.data_ptr(), wsb, st) == 0
        assert handle.pamk_softmax_bwd(xd.data_ptr(), dyd.data_ptr(), dx0.data_ptr(), rows, length, offset, 1, ws.data_ptr(), wsb, st) == 0
        assert handle.pamk_softmax_bwd_saved(e.data_ptr(), dyd.data_ptr(), dx1.data_ptr(), rows, length, offset, 0, 0.0, st) == 0
        assert handle.pamk_softmax_bwd_scaled(xd.data_ptr(), dyd.data_ptr(), dx2.data_ptr(), rows, length, offset, 1, 0.125, ws.data_ptr(), wsb, st) == 0
    assert_bits_equal(y1, y0, "forward with the second output")
    assert_bits_equal(dx1, dx0, "backward from the saved exponentials")
    with _lib.device_guard(dev):
        assert handle.pamk_softmax_bwd_saved(e.data_ptr(), dyd.data_ptr(), dx1.data_ptr(), rows, length, offset, 1, 0.125, st) == 0
    assert_bits_equal(dx1, dx2, "backward from the saved exponentials, scaled")
    assert bool((dx0[0, 0] == 0).all()) and bool(dx0[5].eq(0).all()), "masked entries get no gradient"


@pytest.mark.parametrize("width", [5, 48, 192, 200, 512, 1024])
@pytest.mark.parametrize("affine", [True, False])
def test_layer_norm_backward_from_saved_row_scalars(pam, dev, width, affine):
    """pamk_layer_norm_fwd_save + pamk_layer_norm_bwd_saved against pamk_layer_norm_fwd +
    pamk_layer_norm_bwd(approx): y and dx bit for bit (also for constant rows, whose variance is 0 without
    eps); dweight / dbias are the same per-row terms summed in another order."""
    from pam_b200 import _lib
    handle = _lib.lib()
    g = torch.Generator().manual_seed(width)
    rows = 1001
    x = torch.randn(rows, width, generator=g) * 2 + 0.3
    x[7] = 1.5                                                     # constant row
    dy = torch.randn(rows, width, generator=g)
    w = (torch.randn(width, generator=g).abs() + 0.5).to(dev) if affine else None
    b = torch.randn(width, generator=g).to(dev) if affine else None
    xd, dyd = x.to(dev), dy.to(dev)
    st = _lib.stream_ptr(dev)
    ptr = lambda t: t.data_ptr() if t is not None else None
    wsb = handle.pamk_layer_norm_bwd_workspace_bytes(rows, width)
    ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
    for eps in (1e-5, 0.0):
        y0, y1, dx0, dx1 = (torch.empty_like(xd) for _ in range(4))
        stats = torch.empty(rows, handle.pamk_layer_norm_stats_per_row(), device=dev)
        dw0, db0, dw1, db1 = (torch.empty(width, device=dev) for _ in range(4))
        with _lib.device_guard(dev):
            assert handle.pamk_layer_norm_fwd(xd.data_ptr(), ptr(w), ptr(b), y0.data_ptr(), rows, width, eps, 1.0, st) == 0
            assert handle.pamk_layer_norm_fwd_save(xd.data_ptr(), ptr(w), ptr(b), y1.data_ptr(), stats.data_ptr(), rows, width, eps, 1.0, st) == 0
            assert handle.pamk_layer_norm_bwd(xd.data_ptr(), ptr(w), dyd.data_ptr(), dx0.data_ptr(), ptr(dw0) if affine else None,
                                              db0.data_ptr(), rows, width, eps, 1.0, 1, ws.data_ptr(), wsb, st) == 0
            assert handle.pamk_layer_norm_bwd_saved(xd.data_ptr(), ptr(w), dyd.data_ptr(), stats.data_ptr(), dx1.data_ptr(),
                                                    ptr(dw1) if affine else None, db1.data_ptr(), rows, width, 1.0,
                                                    ws.data_ptr(), wsb, st) == 0
        assert_bits_equal(y1, y0, f"forward with the row scalars, eps={eps}")
        assert_bits_equal(dx1, dx0, f"dx from the saved row scalars, eps={eps}")
        assert_close_nan(db1, db0, 1e-5, 1e-5 * float(db0.nan_to_num().abs().max()), "dbias")
        if affine:      # (without eps the constant row's NaN reaches every column of dweight, on both sides)
            assert_close_nan(dw1, dw0, 1e-5, 1e-5 * float(dw0.nan_to_num().abs().max()), "dweight")
