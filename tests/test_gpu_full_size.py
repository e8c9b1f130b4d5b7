"""The scaling-sweep configuration at its full sizes: square PAM products up to 16384^3 and the
elementwise / pam_ln kernels on 2^28 elements, inputs N(0,1) with 1 % injected special values
(zeros of both signs, denormals, magnitudes 1e30 and 1e-30).

At these sizes the CPU oracle cannot produce the whole result, so each case is checked three ways:
a sample (rows and columns of a product at full K, slices of an elementwise result, rows of a
normalisation) bit for bit against the oracle; a size-independent property (permuting the rows of
A permutes the rows of C; the kernel applied to the whole tensor equals the kernel applied to its
halves); and the input is generated on the device so the test stays within a few seconds."""
import pytest
import torch

from conftest import assert_bits_equal, bits_equal

pytestmark = pytest.mark.gpu

SPECIALS = [0.0, -0.0, 1e-40, -1e-40, 1.4e-45, -1.4e-45, 1e30, -1e30, 1e-30, -1e-30]


@pytest.fixture(scope="module")
def pam():
    import pam_b200
    assert torch.cuda.is_available(), "gpu-marked tests need a CUDA device"
    pam_b200.set_strict_k_order(True)
    yield pam_b200
    pam_b200.set_strict_k_order(False)


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


@pytest.fixture(scope="module")
def K(oracle):
    return oracle.kernels()


def device_randn_with_specials(shape, seed, dev, frac=0.01, values=SPECIALS):
    g = torch.Generator(device=dev).manual_seed(seed)
    t = torch.randn(shape, generator=g, device=dev)
    flat = t.view(-1)
    count = max(1, int(flat.numel() * frac))
    idx = torch.randint(0, flat.numel(), (count,), generator=g, device=dev)
    vals = torch.tensor(values, dtype=torch.float32, device=dev)
    flat[idx] = vals[torch.arange(count, device=dev) % vals.numel()]
    return t


@pytest.mark.parametrize("n", [8192, 16384])
def test_square_gemm_with_specials(pam, K, dev, n):
    A = device_randn_with_specials((n, n), 100 + n, dev)
    B = device_randn_with_specials((n, n), 200 + n, dev)
    ck = pam.cuda_bindings.cuda_kernels
    C = ck.pam_matmul_fwd(A, B, True, True, 1.0)
    g = torch.Generator().manual_seed(n)
    r = torch.randperm(n, generator=g)[:32].to(dev)
    c = torch.randperm(n, generator=g)[:32].to(dev)
    want = K.pam_matmul_fwd(A[r].cpu(), B[:, c].cpu().contiguous())
    assert_bits_equal(C[r][:, c], want, f"sampled block of {n}^3")
    # NaNs (1e30 * 1e30 products) and flushed products must both occur in this input
    assert bool(torch.isnan(C).any()) and bool(torch.isfinite(C).any())
    perm = torch.randperm(n, generator=g).to(dev)
    Cp = ck.pam_matmul_fwd(A[perm], B, True, True, 1.0)
    assert bool(bits_equal(Cp, C[perm]).all())


@pytest.mark.parametrize("log2n", [20, 28])
@pytest.mark.parametrize("op", ["mul", "div"])
def test_elementwise_with_specials(pam, K, dev, op, log2n):
    n = 1 << log2n
    a = device_randn_with_specials((n,), 300 + log2n, dev)
    b = device_randn_with_specials((n,), 400 + log2n, dev)
    fn = pam.mul if op == "mul" else pam.div
    ref = K.pam_fwd if op == "mul" else K.pad_fwd
    out = fn(a, b)
    span = 1 << 18
    for start in (0, n // 2 - span // 2 + 1, n - span):      # the middle slice starts off any vector boundary
        sl = slice(start, start + span)
        assert_bits_equal(out[sl], ref(a[sl].cpu(), b[sl].cpu(), 1.0), f"{op} slice at {start}")
    half = n // 2
    assert bool(bits_equal(out[:half], fn(a[:half], b[:half])).all())
    assert bool(bits_equal(out[half:], fn(a[half:], b[half:])).all())


@pytest.mark.parametrize("huge", [True, False], ids=["all_specials", "no_1e30"])
@pytest.mark.parametrize("width", [192, 512])
def test_layer_norm_2_pow_28_elements(pam, dev, width, huge):
    """pam_ln, forward and backward, on the largest row count that fits 2^28 elements; a sample of
    rows against the CPU replay of the kernel's chain (bit for bit: rows are independent), the
    halves property for y and dx, and the parameter gradients within the tolerance of an fp32 column
    sum over that many rows.  A row that holds 1e30 has a NaN variance (1e30 * 1e30 is outside the
    PAM range), which makes every column sum NaN, so the parameter gradients are checked on the
    input without those two values."""
    import ln_emulation as E
    from test_gpu_parity import _ln_vec
    rows = (1 << 28) // width
    x = device_randn_with_specials((rows, width), 500 + width, dev,
                                   values=SPECIALS if huge else [v for v in SPECIALS if abs(v) < 1e20])
    gy = torch.randn(rows, width, device=dev, generator=torch.Generator(device=dev).manual_seed(width))
    w = torch.rand(width, device=dev) + 0.5
    b = torch.randn(width, device=dev)

    def run(xs, gs):
        xi = xs.clone().requires_grad_()
        wi, bi = w.clone().requires_grad_(), b.clone().requires_grad_()
        y = pam.layer_norm(xi, (width,), wi, bi, 1e-5, approx_bwd=True)
        y.backward(gs)
        return y.detach(), xi.grad, wi.grad, bi.grad

    y, dx, dw, db = run(x, gy)
    g = torch.Generator().manual_seed(width)
    sample = torch.cat([torch.arange(4), torch.randint(0, rows, (56,), generator=g), torch.arange(rows - 4, rows)])
    chain = E.Chain(None, E.kernel_rowsum(_ln_vec(width)), E.torch_colsum)
    wy, wdx, _, _ = chain.run(x[sample.to(dev)].cpu(), w.cpu(), b.cpu(), gy[sample.to(dev)].cpu(), 1e-5, True)
    assert_bits_equal(y[sample.to(dev)], wy, "y rows")
    assert_bits_equal(dx[sample.to(dev)], wdx, "dx rows")
    half = rows // 2
    y0, dx0, dw0, db0 = run(x[:half], gy[:half])
    y1, dx1, dw1, db1 = run(x[half:], gy[half:])
    assert bool(bits_equal(y[:half], y0).all()) and bool(bits_equal(y[half:], y1).all())
    assert bool(bits_equal(dx[:half], dx0).all()) and bool(bits_equal(dx[half:], dx1).all())
    if huge:
        assert bool(torch.isnan(y).any()) and bool(torch.isfinite(y).any())
        return
    # column sums over ~10^6 rows: the two halves add up to the whole within fp32 summation error
    finite = torch.isfinite(db)
    scale = gy.abs().sum(0)
    assert bool(((db - (db0 + db1)).abs()[finite] <= 1e-5 * scale[finite] + 1e-6).all())
    fin_w = torch.isfinite(dw) & torch.isfinite(dw0 + dw1)
    assert bool(((dw - (dw0 + dw1)).abs()[fin_w] <= 1e-4 * (dw.abs()[fin_w] + scale[fin_w])).all())
