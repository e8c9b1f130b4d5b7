"""Parity cases against the fixtures generated from the reference (tests/golden/make_golden.py).

The same functions run in two settings:
  * on CPU tensors over the oracle-backed fake library (tests/cpu_backend.py) — checks the Python
    host layer without a GPU, bit for bit;
  * on CUDA tensors over libpam_b200.so — the parity tests proper (marked gpu).

Tolerances: per-element operations must match the reference bit for bit.  Values that pass
through an ordinary fp32 reduction (torch.sum over a row, the gradient of a broadcast operand,
a matrix product with split-K) may differ by the association of the sum; they are compared with
rtol 2e-5 / atol scaled to the data when `exact_sums` is False.
"""
import math

import torch

from conftest import assert_bits_equal, assert_close_nan

MODES = [(o, a) for o in ("none", "o1") for a in ("exact", "approx")]


def _leaf(t, dev):
    """A fresh leaf tensor on `dev` (``.to`` alone aliases the fixture when dev is the CPU)."""
    return t.to(dev).clone().requires_grad_()


def _off(oname):
    return None if oname == "none" else 1.0552


def _cmp(got, want, what, exact, rtol=2e-5, atol=1e-6):
    if exact:
        assert_bits_equal(got, want, what)
    else:
        assert_close_nan(got, want, rtol, atol, what)


def mul_div(pam, golden, dev, oname, mode):
    for opname, op in (("mul", pam.mul), ("div", pam.div)):
        a = _leaf(golden["ew/a"], dev)
        b = _leaf(golden["ew/b"], dev)
        y = op(a, b, offset=_off(oname), approx_bwd=(mode == "approx"))
        y.backward(golden["ew/dc"].to(dev))
        key = f"ew/{opname}/{oname}/{mode}"
        assert_bits_equal(y, golden[key + "/y"], key)
        assert_bits_equal(a.grad, golden[key + "/da"], key + "/da")
        assert_bits_equal(b.grad, golden[key + "/db"], key + "/db")


def broadcast(pam, golden, dev, exact_sums):
    m = golden["bc/m"].to(dev)
    for opname, op in (("mul", pam.mul), ("div", pam.div)):
        for tag, other, approx in (("row", golden["bc/row"], True), ("col", golden["bc/col"], False)):
            x, z = m.clone().requires_grad_(), _leaf(other, dev)
            y = op(x, z, approx_bwd=approx)
            y.backward(torch.ones_like(y))
            key = f"bc/{opname}/{tag}"
            assert_bits_equal(y, golden[key + "/y"], key)
            assert_bits_equal(x.grad, golden[key + "/d0"], key + "/d0")
            _cmp(z.grad, golden[key + "/d1"], key + "/d1", exact_sums, atol=1e-5)
        x = m.clone().requires_grad_()
        y = op(x, 0.3, approx_bwd=True)
        y.backward(torch.ones_like(y))
        assert_bits_equal(y, golden[f"bc/{opname}/scalar/y"])
        assert_bits_equal(x.grad, golden[f"bc/{opname}/scalar/d0"])
    got = torch.tensor([pam.mul(1.3, -1.3), pam.div(0.1, 9999.0), pam.pow(2.5, 0.5)], dtype=torch.float64)
    assert all(isinstance(v, float) for v in (pam.mul(1.3, -1.3), pam.div(0.1, 9999.0)))
    assert torch.equal(got, golden["bc/scalar_scalar"])


def exp_log(pam, golden, dev, base, oname, mode, log_edges_exact=True):
    bval = {"e": math.e, "2": 2.0, "10": 10.0}[base]
    for opname, op, xin in (("exp", pam.exp, "el/x"), ("log", pam.log, "el/xp")):
        x = _leaf(golden[xin], dev)
        y = op(x, bval, offset=_off(oname), approx_bwd=(mode == "approx"))
        y.backward(golden["ew/dc"].to(dev))
        key = f"el/{opname}/{base}/{oname}/{mode}"
        assert_bits_equal(y, golden[key + "/y"], key)
        assert_bits_equal(x.grad, golden[key + "/dx"], key + "/dx")


def pow_(pam, golden, dev):
    for mode in ("exact", "approx"):
        a = _leaf(golden["pow/a"], dev)
        y = pam.pow(a, 0.5, approx_bwd=(mode == "approx"))
        y.backward(torch.ones_like(y))
        assert_bits_equal(y, golden[f"pow/{mode}/y"])
        assert_bits_equal(a.grad, golden[f"pow/{mode}/dx"])


def matmul(pam, golden, dev, tag, oname, mode, exact_sums=True):
    A = _leaf(golden[f"mm/{tag}/A"], dev)
    B = _leaf(golden[f"mm/{tag}/B"], dev)
    y = pam.matmul(A, B, offset=_off(oname), approx_bwd=(mode == "approx"))
    y.backward(golden[f"mm/{tag}/gC"].to(dev))
    key = f"mm/{tag}/{mode}" if tag != "rand" else f"mm/rand/{oname}/{mode}"
    _cmp(y, golden[key + "/y"], key, exact_sums)
    _cmp(A.grad, golden[key + "/dA"], key + "/dA", exact_sums)
    _cmp(B.grad, golden[key + "/dB"], key + "/dB", exact_sums)


def matmul_layouts(pam, golden, dev):
    """Transposed (column-major) operands must give the same bits as their contiguous copies."""
    A, B = golden["mm/rand/A"].to(dev), golden["mm/rand/B"].to(dev)
    want = golden["mm/rand/none/exact/y"]
    At = A.T.contiguous().T            # contiguous along M
    Bt = B.T.contiguous().T            # contiguous along K
    for a in (A, At):
        for b in (B, Bt):
            assert_bits_equal(pam.matmul(a, b), want, f"layout {a.stride()} x {b.stride()}")
    ab = A.nan_to_num(0, 0, 0), B.nan_to_num(0, 0, 0)
    assert_bits_equal(pam.cuda_bindings.standard_matmul(*ab), golden["mm/rand/standard/y"])


def bmm(pam, golden, dev):
    for mode in ("exact", "approx"):
        A, B = _leaf(golden["bmm/A"], dev), _leaf(golden["bmm/B"], dev)
        y = pam.bmm(A, B, approx_bwd=(mode == "approx"))
        y.backward(golden["bmm/gC"].to(dev))
        assert_bits_equal(y, golden[f"bmm/{mode}/y"])
        assert_bits_equal(A.grad, golden[f"bmm/{mode}/dA"])
        assert_bits_equal(B.grad, golden[f"bmm/{mode}/dB"])


def linear_module(pam, golden, dev, exact_sums):
    lin = pam.Linear(24, 10, approx_bwd=True).to(dev)
    with torch.no_grad():
        lin.weight.copy_(golden["linear/W"])
        lin.bias.copy_(golden["linear/b"])
    X = _leaf(golden["linear/X"], dev)
    y = lin(X)
    y.backward(golden["linear/gy"].to(dev))
    assert_bits_equal(y, golden["linear/y"], "linear/y")
    assert_bits_equal(X.grad, golden["linear/dX"], "linear/dX")
    assert_bits_equal(lin.weight.grad, golden["linear/dW"], "linear/dW")
    _cmp(lin.bias.grad, golden["linear/db"], "linear/db", exact_sums, atol=1e-5)
    assert repr(lin).startswith("pam.Linear(in_features=24, out_features=10")
    assert set(lin.state_dict()) == {"weight", "bias"}


def reductions(pam, golden, dev, oname, mode, exact_sums):
    kw = dict(offset=_off(oname), approx_bwd=(mode == "approx"))
    k = f"{oname}/{mode}"
    g = golden["sm/g"].to(dev)

    def run(fn, xin, gout):
        x = _leaf(golden[xin], dev)
        y = fn(x)
        y.backward(gout)
        return y, x.grad

    for name, fn, xin, gout in (
        ("softmax", lambda t: pam.softmax(t, dim=-1, **kw), "sm/x", g),
        ("softmax_masked", lambda t: pam.softmax(t, dim=-1, **kw), "sm/x_masked", g),
        ("softmax_dim1", lambda t: pam.softmax(t, dim=1, **kw), "sm/x", g),
        ("log_softmax", lambda t: pam.log_softmax(t, dim=-1, **kw), "sm/x", g),
        ("logsumexp", lambda t: pam.logsumexp(t, dim=-1, **kw), "sm/x", g[..., 0]),
        ("mean", lambda t: pam.mean(t, dim=-1, keepdim=True, **kw), "sm/x", g[..., :1]),
    ):
        y, dx = run(fn, xin, gout)
        _cmp(y, golden[f"sm/{name}/{k}/y"], f"{name}/{k}", exact_sums, rtol=1e-4, atol=1e-6)
        _cmp(dx, golden[f"sm/{name}/{k}/dx"], f"{name}/{k}/dx", exact_sums, rtol=2e-3, atol=2e-5)


def layer_norm(pam, golden, dev, oname, mode, exact_sums):
    kw = dict(offset=_off(oname), approx_bwd=(mode == "approx"))
    k = f"{oname}/{mode}"
    x = _leaf(golden["ln/x"], dev)
    w, b = _leaf(golden["ln/w"], dev), _leaf(golden["ln/b"], dev)
    y = pam.layer_norm(x, 48, w, b, 1e-5, **kw)
    y.backward(golden["ln/g"].to(dev))
    for name, val, rtol, atol in (("y", y, 1e-4, 1e-5), ("dx", x.grad, 2e-3, 2e-4), ("dw", w.grad, 2e-3, 2e-4),
                                  ("db", b.grad, 1e-4, 1e-5)):
        _cmp(val, golden[f"ln/affine/{k}/{name}"], f"ln/affine/{k}/{name}", exact_sums, rtol=rtol, atol=atol)
    x = _leaf(golden["ln/x"], dev)
    y = pam.layer_norm(x, (48,), None, None, 1e-6, **kw)
    y.backward(golden["ln/g"].to(dev))
    _cmp(y, golden[f"ln/plain/{k}/y"], "ln/plain/y", exact_sums, rtol=1e-4, atol=1e-5)
    _cmp(x.grad, golden[f"ln/plain/{k}/dx"], "ln/plain/dx", exact_sums, rtol=2e-3, atol=2e-4)


def cross_entropy(pam, factories, golden, dev, exact_sums):
    ops = factories.get_function_dict('{"type": "pam", "dkwargs": {"approx_bwd": true}}')
    for ls in (0.0, 0.1):
        x = _leaf(golden["ce/x"], dev)
        y = pam.cross_entropy(x, golden["ce/t"].to(dev), None, 1, "mean", ls, op_dict=ops)
        y.backward()
        assert_close_nan(y.reshape(1), golden[f"ce/ls{ls}/y"].reshape(1), 1e-5, 1e-6, "ce value")
        _cmp(x.grad, golden[f"ce/ls{ls}/dx"], "ce grad", exact_sums, rtol=1e-4, atol=1e-6)


def adam(optim, golden, dev, exact_sums=True):
    p = torch.nn.Parameter(golden["adam/p0"].to(dev).clone())
    opt = optim.Adam([p], lr=5e-4, betas=(0.9, 0.98), eps=1e-8, weight_decay=1e-4, opt_functional_cfg="pam")
    for step in (1, 2, 3):
        p.grad = golden[f"adam/g{step}"].to(dev).clone()
        opt.step()
        st = opt.state[p]
        assert st["step"] == step
        assert_bits_equal(st["exp_avg"], golden[f"adam/m{step}"], f"adam m{step}")
        assert_bits_equal(st["exp_avg_sq"], golden[f"adam/v{step}"], f"adam v{step}")
        assert_bits_equal(p.detach(), golden[f"adam/p{step}"], f"adam p{step}")
