"""CPU checks of the oracle itself: the C restatement against the reference's known-answer
vectors (pam/test_pam.py) and against fixtures produced by the reference's own code
(tests/golden/make_golden.py)."""
import math

import pytest
import torch

from conftest import assert_bits_equal


def test_reference_known_answers(oracle):
    # the 15 (a, b, expected) triples of the reference's pam_fwd_test, pam/test_pam.py:13-29
    abc = torch.tensor([
        [1.0, 1.0, 1.0], [1.2345, 1.0, 1.2345], [1.2345, 32.0, 32.0 * 1.2345],
        [-1.2345, 32.0, -32.0 * 1.2345], [1.2345, -32.0, -32.0 * 1.2345], [-1.2345, -32.0, 32.0 * 1.2345],
        [1.0, 0.0, 0.0], [0.0, -1.0, -0.0], [1.5, 1.5, 2.0], [1.3, -1.3, -1.6],
        [4.5, 3.0, 8 * (1 + (4.5 - 4) / 4 + (3.0 - 2) / 2)], [-6.0, 3.0, -16.0],
        [-3.5, -3.5, 8 * (1 + (3.5 - 2) / 2 + (3.5 - 2) / 2 - 1)], [1e-30, 1e-30, 0.0], [1e-30, -1e-30, -0.0],
    ])
    got = oracle.kernels().pam_fwd(abc[:, 0].contiguous(), abc[:, 1].contiguous(), 1.0)
    assert torch.allclose(abc[:, 2], got)
    # the integer formulation returns +0.0 for every flushed product, whatever the signs
    assert got[[6, 7, 13, 14]].view(torch.int32).eq(0).all()


def test_reference_inf_nan_vectors(oracle):
    # pam/test_pam.py:36-43; the CUDA semantics return NaN (never +-inf) for all six
    ab = torch.tensor([[1e30, 1e30], [1e30, -1e30], [float("-inf"), 1e-20], [float("nan"), -1e-20],
                       [float("inf"), 0.0], [float("nan"), 0.0]])
    got = oracle.kernels().pam_fwd(ab[:, 0].contiguous(), ab[:, 1].contiguous(), 1.0)
    assert got.isnan().all()


def test_threshold_bit_patterns(oracle):
    # |a*b| is compared with the double literals 1e-37 / 1e37: flush iff bits <= 0x02081CEA,
    # pass iff bits <= 0x7CF0BDC2.
    K = oracle.kernels()
    t = torch.tensor([0x02081CEA, 0x02081CEB, 0x7CF0BDC2, 0x7CF0BDC3], dtype=torch.int32).view(torch.float32)
    got = K.pam_fwd(t, torch.ones(4), 1.0)
    assert got[0].item() == 0.0 and got[1].item() == t[1].item()
    assert got[2].item() == t[2].item() and math.isnan(got[3].item())


def test_exact_gradient_recipe(oracle):
    # pam/test_pam.py:48-73: exact backward equals the analytic power-of-two slope
    g = torch.Generator().manual_seed(1)
    n = 128
    A = (2.0 ** torch.randint(-30, 30, (n,), generator=g)) * (1 + torch.rand(n, generator=g))
    B = (2.0 ** torch.randint(-30, 30, (n,), generator=g)) * (1 + torch.rand(n, generator=g))
    dC = torch.arange(n).float()
    A1, B1 = A.clone().requires_grad_(), B.clone().requires_grad_()
    oracle.mul(A1, B1).backward(dC)
    fa, ea = torch.frexp(A)                                # A = fa * 2^ea, fa in [0.5, 1)
    fb, eb = torch.frexp(B)
    carry = ((fa * 2 - 1) + (fb * 2 - 1)) >= 1.0           # mantissa fractions sum past 1
    assert torch.equal(A1.grad, dC * torch.exp2((eb - 1 + carry).float()))
    assert torch.equal(B1.grad, dC * torch.exp2((ea - 1 + carry).float()))


CASES_EW = [(o, a) for o in ("none", "o1") for a in ("exact", "approx")]


@pytest.mark.parametrize("oname,mode", CASES_EW)
def test_mul_div_against_reference(oracle, golden, oname, mode):
    off = None if oname == "none" else 1.0552
    for opname, op in (("mul", oracle.mul), ("div", oracle.div)):
        a, b = golden["ew/a"].clone().requires_grad_(), golden["ew/b"].clone().requires_grad_()
        y = op(a, b, offset=off, approx_bwd=(mode == "approx"))
        y.backward(golden["ew/dc"])
        key = f"ew/{opname}/{oname}/{mode}"
        assert_bits_equal(y, golden[key + "/y"], key)
        assert_bits_equal(a.grad, golden[key + "/da"], key + "/da")
        assert_bits_equal(b.grad, golden[key + "/db"], key + "/db")


@pytest.mark.parametrize("base", ["e", "2", "10"])
@pytest.mark.parametrize("oname,mode", CASES_EW)
def test_exp_log_against_reference(oracle, golden, base, oname, mode):
    off = None if oname == "none" else 1.0552
    bval = {"e": math.e, "2": 2.0, "10": 10.0}[base]
    for opname, op, xin in (("exp", oracle.exp, "el/x"), ("log", oracle.log, "el/xp")):
        x = golden[xin].clone().requires_grad_()
        y = op(x, bval, offset=off, approx_bwd=(mode == "approx"))
        y.backward(golden["ew/dc"])
        key = f"el/{opname}/{base}/{oname}/{mode}"
        assert_bits_equal(y, golden[key + "/y"], key)
        assert_bits_equal(x.grad, golden[key + "/dx"], key + "/dx")


@pytest.mark.parametrize("tag", ["ref21", "ref20", "rand"])
@pytest.mark.parametrize("mode", ["exact", "approx"])
def test_matmul_against_reference(oracle, golden, tag, mode):
    A, B = golden[f"mm/{tag}/A"].clone().requires_grad_(), golden[f"mm/{tag}/B"].clone().requires_grad_()
    y = oracle.matmul(A, B, approx_bwd=(mode == "approx"))
    y.backward(golden[f"mm/{tag}/gC"])
    key = f"mm/{tag}/{mode}" if tag != "rand" else f"mm/rand/none/{mode}"
    assert_bits_equal(y, golden[key + "/y"], key)
    assert_bits_equal(A.grad, golden[key + "/dA"], key + "/dA")
    assert_bits_equal(B.grad, golden[key + "/dB"], key + "/dB")


def test_bmm_and_standard_against_reference(oracle, golden):
    for mode in ("exact", "approx"):
        A, B = golden["bmm/A"].clone().requires_grad_(), golden["bmm/B"].clone().requires_grad_()
        y = oracle.bmm(A, B, approx_bwd=(mode == "approx"))
        y.backward(golden["bmm/gC"])
        assert_bits_equal(y, golden[f"bmm/{mode}/y"])
        assert_bits_equal(A.grad, golden[f"bmm/{mode}/dA"])
        assert_bits_equal(B.grad, golden[f"bmm/{mode}/dB"])
    A = golden["mm/rand/A"].nan_to_num(0, 0, 0)
    B = golden["mm/rand/B"].nan_to_num(0, 0, 0)
    assert_bits_equal(oracle.standard_matmul(A, B), golden["mm/rand/standard/y"])


@pytest.mark.parametrize("oname,mode", CASES_EW)
def test_composites_against_reference(oracle, golden, oname, mode):
    kw = dict(offset=None if oname == "none" else 1.0552, approx_bwd=(mode == "approx"))
    k = f"{oname}/{mode}"
    g = golden["sm/g"]

    def run(fn, xin, gout):
        x = golden[xin].clone().requires_grad_()
        y = fn(x)
        y.backward(gout)
        return y, x.grad

    for name, fn, xin, gout in (
        ("softmax", lambda t: oracle.softmax(t, dim=-1, **kw), "sm/x", g),
        ("softmax_masked", lambda t: oracle.softmax(t, dim=-1, **kw), "sm/x_masked", g),
        ("softmax_dim1", lambda t: oracle.softmax(t, dim=1, **kw), "sm/x", g),
        ("log_softmax", lambda t: oracle.log_softmax(t, dim=-1, **kw), "sm/x", g),
        ("logsumexp", lambda t: oracle.logsumexp(t, dim=-1, **kw), "sm/x", g[..., 0]),
        ("mean", lambda t: oracle.mean(t, dim=-1, keepdim=True, **kw), "sm/x", g[..., :1]),
    ):
        y, dx = run(fn, xin, gout)
        assert_bits_equal(y, golden[f"sm/{name}/{k}/y"], f"{name}/{k}")
        assert_bits_equal(dx, golden[f"sm/{name}/{k}/dx"], f"{name}/{k}/dx")

    x = golden["ln/x"].clone().requires_grad_()
    w, b = golden["ln/w"].clone().requires_grad_(), golden["ln/b"].clone().requires_grad_()
    y = oracle.layer_norm(x, 48, w, b, 1e-5, **kw)
    y.backward(golden["ln/g"])
    for name, val in (("y", y), ("dx", x.grad), ("dw", w.grad), ("db", b.grad)):
        assert_bits_equal(val, golden[f"ln/affine/{k}/{name}"], f"ln/affine/{k}/{name}")
    x = golden["ln/x"].clone().requires_grad_()
    y = oracle.layer_norm(x, (48,), None, None, 1e-6, **kw)
    y.backward(golden["ln/g"])
    assert_bits_equal(y, golden[f"ln/plain/{k}/y"])
    assert_bits_equal(x.grad, golden[f"ln/plain/{k}/dx"])


def test_pow_and_adam_against_reference(oracle, golden):
    for mode in ("exact", "approx"):
        a = golden["pow/a"].clone().requires_grad_()
        y = oracle.pow(a, 0.5, approx_bwd=(mode == "approx"))
        y.backward(torch.ones_like(y))
        assert_bits_equal(y, golden[f"pow/{mode}/y"])
        assert_bits_equal(a.grad, golden[f"pow/{mode}/dx"])
    p = golden["adam/p0"]
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    for step in (1, 2, 3):
        p, m, v = oracle.adam_step(p, golden[f"adam/g{step}"], m, v, step=step, lr=5e-4, betas=(0.9, 0.98),
                                   eps=1e-8, weight_decay=1e-4)
        assert_bits_equal(p, golden[f"adam/p{step}"], f"adam p step {step}")
        assert_bits_equal(m, golden[f"adam/m{step}"])
        assert_bits_equal(v, golden[f"adam/v{step}"])


@pytest.mark.parametrize("oname,mode", CASES_EW)
def test_fused_layer_norm_chain_equals_reference(oracle, golden, oname, mode):
    """The primitive-by-primitive chain that the fused pam_ln kernel evaluates (tests/ln_emulation.py),
    summed with torch.sum, is the reference's layer_norm forward and backward bit for bit."""
    import ln_emulation as E
    chain = E.Chain(None if oname == "none" else 1.0552, E.torch_rowsum, E.torch_colsum)
    approx = mode == "approx"
    k = f"{oname}/{mode}"
    y, dx, dw, db = chain.run(golden["ln/x"], golden["ln/w"], golden["ln/b"], golden["ln/g"], 1e-5, approx)
    assert_bits_equal(y.view(7, 3, 48), golden[f"ln/affine/{k}/y"])
    assert_bits_equal(dx.view(7, 3, 48), golden[f"ln/affine/{k}/dx"])
    assert_bits_equal(dw, golden[f"ln/affine/{k}/dw"])
    assert_bits_equal(db, golden[f"ln/affine/{k}/db"])
    y, dx, _, _ = chain.run(golden["ln/x"], None, None, golden["ln/g"], 1e-6, approx)
    assert_bits_equal(y.view(7, 3, 48), golden[f"ln/plain/{k}/y"])
    assert_bits_equal(dx.view(7, 3, 48), golden[f"ln/plain/{k}/dx"])


@pytest.mark.parametrize("oname,mode", CASES_EW)
def test_fused_softmax_chain_equals_reference(oracle, golden, oname, mode):
    """The chains that the fused softmax / logsumexp kernels evaluate, summed with torch.sum, are the
    reference's softmax, logsumexp and log_softmax forward and backward bit for bit."""
    import ln_emulation as E
    chain = E.Chain(None if oname == "none" else 1.0552, E.torch_rowsum, E.torch_colsum)
    approx = mode == "approx"
    k = f"{oname}/{mode}"
    g = golden["sm/g"]
    for name, xin in (("softmax", "sm/x"), ("softmax_masked", "sm/x_masked")):
        y, dx = chain.softmax(golden[xin], g, approx)
        assert_bits_equal(y.view(6, 5, 11), golden[f"sm/{name}/{k}/y"], name)
        assert_bits_equal(dx.view(6, 5, 11), golden[f"sm/{name}/{k}/dx"], name + "/dx")
    y, dx = chain.logsumexp(golden["sm/x"], g[..., 0], approx)
    assert_bits_equal(y.view(6, 5), golden[f"sm/logsumexp/{k}/y"], "logsumexp")
    assert_bits_equal(dx.view(6, 5, 11), golden[f"sm/logsumexp/{k}/dx"], "logsumexp/dx")
    # log_softmax = x - logsumexp(keepdim): its gradient is g - d(logsumexp)(sum of g over the row)
    y, dlse = chain.logsumexp(golden["sm/x"], -g.sum(-1), approx)
    assert_bits_equal(golden["sm/x"] - y.view(6, 5, 1), golden[f"sm/log_softmax/{k}/y"], "log_softmax")
    assert_bits_equal(g + dlse.view(6, 5, 11), golden[f"sm/log_softmax/{k}/dx"], "log_softmax/dx")
