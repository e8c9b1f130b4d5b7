"""The Python host layer (operand description, broadcasting, autograd pairing, modules, factories,
optimizer) over the oracle-backed fake library, against fixtures generated from the reference.
No GPU is needed; the CUDA kernels themselves are checked by the gpu-marked tests."""
import pytest
import torch

import cpu_backend
import parity_cases as cases

import pam_b200 as pam
from pam_b200 import factories, optim

DEV = torch.device("cpu")


@pytest.fixture()
def backend(monkeypatch, oracle):
    return cpu_backend.install(monkeypatch)


@pytest.mark.parametrize("oname,mode", cases.MODES)
def test_mul_div(backend, golden, oname, mode):
    cases.mul_div(pam, golden, DEV, oname, mode)


def test_broadcast_operands_are_not_materialised(backend, golden):
    cases.broadcast(pam, golden, DEV, exact_sums=True)
    kinds = {tuple(c[1]) for c in backend.calls if c[0] in ("orc_pam", "orc_pad")}
    assert (0, 2) in kinds and (0, 3) in kinds and (0, 4) in kinds       # FULL x ROW / COL / IMM


@pytest.mark.parametrize("base", ["e", "2", "10"])
@pytest.mark.parametrize("oname,mode", cases.MODES)
def test_exp_log(backend, golden, base, oname, mode):
    cases.exp_log(pam, golden, DEV, base, oname, mode)


def test_pow(backend, golden):
    cases.pow_(pam, golden, DEV)


@pytest.mark.parametrize("tag,oname", [("ref21", "none"), ("ref20", "none"), ("rand", "none"), ("rand", "o1")])
@pytest.mark.parametrize("mode", ["exact", "approx"])
def test_matmul(backend, golden, tag, oname, mode):
    cases.matmul(pam, golden, DEV, tag, oname, mode)


def test_matmul_layouts_and_bmm(backend, golden):
    cases.matmul_layouts(pam, golden, DEV)
    cases.bmm(pam, golden, DEV)
    # transposed operands reach the library as strides, not copies
    mm = [c for c in backend.calls if c[0] == "matmul"]
    assert any(c[3][1] == 1 and c[3][2] != 1 for c in mm) and any(c[4][1] == 1 and c[4][2] != 1 for c in mm)


def test_linear_module(backend, golden):
    cases.linear_module(pam, golden, DEV, exact_sums=True)


@pytest.mark.parametrize("oname,mode", cases.MODES)
def test_reductions_and_layer_norm(backend, golden, oname, mode):
    cases.reductions(pam, golden, DEV, oname, mode, exact_sums=True)
    cases.layer_norm(pam, golden, DEV, oname, mode, exact_sums=True)


def test_cross_entropy(backend, golden):
    cases.cross_entropy(pam, factories, golden, DEV, exact_sums=True)


def test_adam(backend, golden):
    cases.adam(optim, golden, DEV)


def test_cpu_tensors_are_refused_without_the_fake_backend():
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        pam.mul(torch.ones(3), torch.ones(3))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        pam.matmul(torch.ones(3, 3), torch.ones(3, 3))


def test_conv_power_of_two_equivalence(backend):
    # the reference's recipe (pam/test_pam.py:151-195): with power-of-two weights PAM == multiply
    g = torch.Generator().manual_seed(7)
    X = (torch.randint(-1024, 1024, (3, 5, 9, 8), generator=g) / 64.0).requires_grad_()
    W = (2.0 ** torch.randint(-8, 8, (7, 5, 3, 5), generator=g)).requires_grad_()
    X2, W2 = X.detach().clone().requires_grad_(), W.detach().clone().requires_grad_()
    Y = pam.conv2d(X, W, approx_bwd=True)
    Y.sum().backward()
    Y2 = torch.nn.functional.conv2d(X2, W2)
    Y2.sum().backward()
    close = lambda u, v: torch.allclose(u, v, rtol=1e-5, atol=1e-3)   # fp32 sums in a different order
    assert close(Y, Y2) and close(X.grad, X2.grad) and close(W.grad, W2.grad)
    for G in (1, 4):
        X = (torch.randint(-8, 9, (3, 8, 7, 9), generator=g) / 4.0).requires_grad_()
        W = (2.0 ** torch.randint(-2, 3, (16, 8 // G, 3, 5), generator=g)).requires_grad_()
        X2, W2 = X.detach().clone().requires_grad_(), W.detach().clone().requires_grad_()
        Y = pam.conv2d_group(X, W, groups=G, approx_bwd=True)
        Y.sum().backward()
        Y2 = torch.nn.functional.conv2d(X2, W2, groups=G)
        Y2.sum().backward()
        assert close(Y, Y2) and close(X.grad, X2.grad) and close(W.grad, W2.grad)
    conv = pam.Conv2d(5, 7, (3, 5), padding="same", approx_bwd=True)
    assert conv(torch.randn(2, 5, 6, 6, generator=g)).shape == (2, 7, 6, 6)
    assert repr(conv).startswith("pam.Conv2d(5, 7")


def test_patch_convolution_without_unfold_equals_unfold_route(backend):
    """Non-overlapping patches (stride = kernel: a ViT patch embedding) skip F.unfold; values and
    gradients must be those of the reference's unfold + linear route (pam/pam_ops.py:118-161)."""
    g = torch.Generator().manual_seed(8)
    X = torch.randn(2, 3, 32, 48, generator=g)
    W = torch.randn(5, 3, 16, 16, generator=g) * 0.1
    b = torch.randn(5, generator=g)
    gy = torch.randn(2, 5, 2, 3, generator=g)

    def unfold_route(x, w, bias):
        cols = torch.nn.functional.unfold(x, (16, 16), stride=16)
        y = pam.linear(cols.transpose(1, 2).reshape(-1, cols.shape[1]), w.view(5, -1), approx_bwd=True)
        return y.view(2, -1, 5).transpose(1, 2).reshape(2, 5, 2, 3) + bias.view(1, -1, 1, 1)

    outs = []
    for route in (lambda x, w, bias: pam.conv2d(x, w, bias, stride=16, approx_bwd=True), unfold_route):
        x, w, bias = (t.clone().requires_grad_() for t in (X, W, b))
        y = route(x, w, bias)
        y.backward(gy)
        outs.append((y.detach(), x.grad, w.grad, bias.grad))
    for name, got, want in zip(("y", "dx", "dw", "db"), *outs):
        assert torch.equal(got, want), name


@pytest.mark.parametrize("approx", [True, False])
def test_linear_with_bias_in_the_epilogue_equals_product_plus_add(backend, approx):
    """The autograd function behind the fused `linear` (bias added by the product's epilogue, bias
    gradient by the column-sum entry point) against the reference's composition, product then add."""
    from pam_b200 import cuda_bindings as cb
    g = torch.Generator().manual_seed(21)
    X, W, b, gy = (torch.randn(9, 14, generator=g), torch.randn(6, 14, generator=g), torch.randn(6, generator=g),
                   torch.randn(9, 6, generator=g))
    outs = []
    for route in (lambda x, w, bias: cb.pam_linear(x, w, bias, approx_bwd=approx),
                  lambda x, w, bias: pam.matmul(x, w.T, approx_bwd=approx) + bias):
        x, w, bias = (t.clone().requires_grad_() for t in (X, W, b))
        y = route(x, w, bias)
        y.backward(gy)
        outs.append((y.detach(), x.grad, w.grad, bias.grad))
    for name, got, want in zip(("y", "dx", "dw", "db"), *outs):
        assert torch.equal(got, want), name
    assert any(c[0] == "matmul" for c in backend.calls)
