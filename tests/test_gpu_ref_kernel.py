"""Bit-for-bit comparison with the reference's own CUDA kernels running on the same GPU.

``baseline/build_ref.py`` compiles the reference's pam/cuda_kernels.cu for sm_100a (with the ten
``.type()`` -> ``.scalar_type()`` substitutions it needs against current PyTorch) into
``baseline/_ref/pam_ref_cuda_kernels.so``.  Where that file exists these tests compare whole
outputs — not samples — of every kernel family with it: a 4096^3 PAM product with 1 % injected
special values, the four operand layouts, batched products, the exact-gradient products (including
offsets below one and K that is not a multiple of the reference's 32-wide tile, where the
reference's zero-filled tail is visible in the result) and the eight elementwise kernels.
Skipped when the reference build is absent."""
import pytest
import torch

from conftest import ROOT, assert_bits_equal

pytestmark = pytest.mark.gpu

SPECIALS = [0.0, -0.0, 1e-40, -1e-40, 1.4e-45, -1.4e-45, 1e30, -1e30, 1e-30, -1e-30]


@pytest.fixture(scope="module")
def ref():
    import sys
    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    from baseline import build_ref
    mod = build_ref.load()
    if mod is None:
        pytest.skip("reference CUDA kernels were not built (baseline/_ref/pam_ref_cuda_kernels.so)")
    return mod


@pytest.fixture(scope="module")
def ours():
    import pam_b200
    assert torch.cuda.is_available(), "gpu-marked tests need a CUDA device"
    pam_b200.set_strict_k_order(True)          # one thread sums each output in k order, as the reference does
    yield pam_b200.cuda_bindings.cuda_kernels
    pam_b200.set_strict_k_order(False)


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


def randn_with_specials(shape, seed, dev, frac=0.01, values=SPECIALS):
    g = torch.Generator(device=dev).manual_seed(seed)
    t = torch.randn(shape, generator=g, device=dev)
    flat = t.view(-1)
    count = max(1, int(flat.numel() * frac))
    idx = torch.randint(0, flat.numel(), (count,), generator=g, device=dev)
    vals = torch.tensor(values, dtype=torch.float32, device=dev)
    flat[idx] = vals[torch.arange(count, device=dev) % vals.numel()]
    return t


def flags(t):
    return t.stride(-1) == 1


def layout(t, column_major):
    return t.mT.contiguous().mT if column_major else t.contiguous()


@pytest.mark.parametrize("frac", [0.01, 0.0, 0.5])
def test_whole_4096_product_with_specials(ref, ours, dev, frac):
    """Every one of the 16.7 M outputs of a 4096^3 product, K order and special handling included."""
    n = 4096
    values = SPECIALS if frac < 0.5 else [0.0]          # 50 % zeros: an activation after ReLU
    A = randn_with_specials((n, n), 11, dev, frac, values) if frac else torch.randn(n, n, device=dev)
    B = randn_with_specials((n, n), 12, dev, frac, values) if frac else torch.randn(n, n, device=dev)
    want = ref.pam_matmul_fwd(A, B, True, True, 1.0)
    got = ours.pam_matmul_fwd(A, B, True, True, 1.0)
    torch.cuda.synchronize()
    assert_bits_equal(got, want, f"4096^3 product, {frac:.0%} specials")
    if frac == 0.01:
        assert bool(torch.isnan(want).any()) and bool(torch.isfinite(want).any())


@pytest.mark.parametrize("a_cm,b_cm", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("offset", [1.0, 1.0552])
def test_layouts_and_ragged_sizes(ref, ours, dev, a_cm, b_cm, offset):
    for (M, K, N) in ((197, 192, 576), (333, 77, 130), (5, 4, 3), (1000, 1030, 64)):
        A = layout(randn_with_specials((M, K), M + K, dev, 0.02), a_cm)
        B = layout(randn_with_specials((K, N), K + N, dev, 0.02), b_cm)
        want = ref.pam_matmul_fwd(A, B, flags(A), flags(B), offset)
        got = ours.pam_matmul_fwd(A, B, flags(A), flags(B), offset)
        assert_bits_equal(got, want, f"{M}x{K}x{N} a_cm={a_cm} b_cm={b_cm} offset={offset}")
        want = ref.standard_matmul(A, B, flags(A), flags(B), 1.0)
        got = ours.standard_matmul(A, B, flags(A), flags(B), 1.0)
        assert_bits_equal(got, want, f"true-multiply {M}x{K}x{N}")


def test_batched_attention_shapes(ref, ours, dev):
    q = randn_with_specials((36, 197, 64), 5, dev, 0.005)
    k = randn_with_specials((36, 197, 64), 6, dev, 0.005)
    kt = k.transpose(1, 2)
    want = ref.pam_bmm_fwd(q, kt, flags(q), flags(kt), 1.0)
    got = ours.pam_bmm_fwd(q, kt, flags(q), flags(kt), 1.0)
    assert_bits_equal(got, want, "q k^T")
    p = torch.softmax(want.nan_to_num(0.0), -1)
    want2 = ref.pam_bmm_fwd(p, q, True, True, 1.0)
    got2 = ours.pam_bmm_fwd(p, q, True, True, 1.0)
    assert_bits_equal(got2, want2, "p v")


@pytest.mark.parametrize("offset", [1.0, 1.0552, 0.97])
@pytest.mark.parametrize("delta_l", [True, False])
def test_exact_gradient_products(ref, ours, dev, offset, delta_l):
    """K values that are and are not multiples of 32: the reference's kernel also accumulates the
    zero-filled tail of its last 32-wide tile, which shows in the result when the offset is below
    one (a padded term is 0 * -inf = NaN for outputs whose D has a small mantissa) or when every
    real term is -0."""
    from pam_b200 import _lib
    lib = _lib.lib()
    for (M, K, N) in ((64, 32, 48), (33, 16, 20), (40, 24, 64), (130, 100, 70), (17, 8, 9), (256, 600, 192)):
        L = torch.randn(M, K, device=dev)
        R = torch.randn(K, N, device=dev)
        D = torch.randn(M, N, device=dev)
        D.view(-1)[::7] = 1.0 + 2.0 ** -20            # small mantissas: offset 0.97 makes the padded slope -inf
        want = ref.pam_matmul_bwd(L, R, D, True, True, delta_l, offset)
        for policy in (0, 1, 2):
            _lib.check(lib.pamk_test_set_tile_policy(policy), "tile policy")
            try:
                got = ours.pam_matmul_bwd(L, R, D, True, True, delta_l, offset)
            finally:
                lib.pamk_test_set_tile_policy(0)
            assert_bits_equal(got, want, f"exact gradient {M}x{K}x{N} offset={offset} delta_l={delta_l} tile policy {policy}")


def test_elementwise_kernels(ref, ours, dev):
    n = (1 << 20) + 3
    a = randn_with_specials((n,), 21, dev, 0.02)
    b = randn_with_specials((n,), 22, dev, 0.02)
    d = randn_with_specials((n,), 23, dev, 0.02)
    for offset in (1.0, 1.0552, 0.97):
        assert_bits_equal(ours.pam_fwd(a, b, offset), ref.pam_fwd(a, b, offset), f"pam_fwd {offset}")
        assert_bits_equal(ours.pam_bwd(a, b, d, offset), ref.pam_bwd(a, b, d, offset), f"pam_bwd {offset}")
        assert_bits_equal(ours.pad_fwd(a, b, offset), ref.pad_fwd(a, b, offset), f"pad_fwd {offset}")
        assert_bits_equal(ours.pad_bwd(a, b, d, offset), ref.pad_bwd(a, b, d, offset), f"pad_bwd {offset}")
    x = torch.randn(n, device=dev) * 8
    pos = torch.rand(n, device=dev) * 100 + 1e-6
    pos[:4096] = 2.0 ** torch.arange(-40, 24, device=dev).repeat(64).float()      # exact powers of two
    for base in (2.0, 2.718281828459045, 10.0):
        assert_bits_equal(ours.pa_exp_fwd(x, base, 1.0), ref.pa_exp_fwd(x, base, 1.0), f"pa_exp_fwd base {base}")
        assert_bits_equal(ours.pa_exp_bwd(x, d, base, 1.0), ref.pa_exp_bwd(x, d, base, 1.0), f"pa_exp_bwd base {base}")
        assert_bits_equal(ours.pa_log_fwd(pos, base, 1.0), ref.pa_log_fwd(pos, base, 1.0), f"pa_log_fwd base {base}")
        assert_bits_equal(ours.pa_log_bwd(pos, d, base, 1.0), ref.pa_log_bwd(pos, d, base, 1.0), f"pa_log_bwd base {base}")
