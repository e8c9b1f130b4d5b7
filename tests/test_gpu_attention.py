"""Attention over a fused q/k/v projection on strided views (``fused.attention_qkv``) against the chain
it replaces — flatten copies, ``bmm``, PAM scaling, PAM softmax, ``bmm``, transpose copy, as the timm
fork's attention module runs it (timm/models/vision_transformer.py:72-93) — and against the oracle.

The strided route issues the same products with the same shapes and split-K plans, scales in the score
product's epilogue with the same scalar function and uses the same softmax kernel, so forward output and
the gradient of qkv must equal the chain bit for bit; against the CPU oracle's composition the sums
associate differently (tolerance stated at the check).
"""
import pytest
import torch

from conftest import assert_bits_equal, assert_close_nan

pytestmark = pytest.mark.gpu

KW = dict(approx_bwd=True)


def chain(ops, qkv, heads, scale, kw):
    B, N, C3 = qkv.shape
    C = C3 // 3
    t = qkv.reshape(B, N, 3, heads, C // heads).permute(2, 0, 3, 1, 4)
    q, k, v = t.unbind(0)
    attn = ops.bmm(q.flatten(0, 1), k.transpose(-2, -1).flatten(0, 1), **kw)
    attn = ops.softmax(ops.mul(attn, scale, **kw), dim=-1, **kw)
    x = ops.bmm(attn, v.flatten(0, 1), **kw).view(B, heads, N, C // heads)
    return x.transpose(1, 2).reshape(B, N, C)


@pytest.mark.parametrize("B,N,heads,hd", [(3, 197, 3, 64), (2, 32, 4, 16), (1, 5, 2, 4), (2, 7, 3, 5), (64, 197, 3, 64), (5, 50, 8, 32)])
@pytest.mark.parametrize("offset", [None, 1.0552])
def test_strided_attention_equals_the_chain_bit_for_bit(B, N, heads, hd, offset):
    import pam_b200 as pam
    from pam_b200 import fused
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(B * 1000 + N)
    C = heads * hd
    qkv0 = torch.randn(B, N, 3 * C, generator=g).to(dev)
    dout = torch.randn(B, N, C, generator=g).to(dev)
    scale = hd ** -0.5
    kw = dict(KW, offset=offset)
    assert fused.attention_supported(qkv0, heads, True)
    a = qkv0.clone().requires_grad_()
    ya = fused.attention_qkv(a, heads, scale, offset=offset)
    ya.backward(dout)
    b = qkv0.clone().requires_grad_()
    yb = chain(pam, b, heads, scale, kw)
    yb.backward(dout)
    assert_bits_equal(ya, yb, "context")
    assert_bits_equal(a.grad, b.grad, "d qkv")


def test_strided_attention_against_the_oracle(oracle):
    from pam_b200 import fused
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(5)
    B, N, heads, hd = 2, 23, 3, 8
    C = heads * hd
    qkv0 = torch.randn(B, N, 3 * C, generator=g)
    dout = torch.randn(B, N, C, generator=g)
    a = qkv0.to(dev).requires_grad_()
    ya = fused.attention_qkv(a, heads, hd ** -0.5)
    ya.backward(dout.to(dev))
    b = qkv0.clone().requires_grad_()
    yb = chain(oracle, b, heads, hd ** -0.5, KW)
    yb.backward(dout)
    # sums of 8 (scores), 23 (softmax rows, context) terms: the GPU adds in k order, torch's CPU sums in blocks
    assert_close_nan(ya.detach(), yb.detach(), 1e-5, 1e-5 * float(yb.detach().abs().max()), "context")
    assert_close_nan(a.grad, b.grad, 1e-4, 1e-4 * float(b.grad.abs().max()), "d qkv")


def test_unsupported_calls_are_refused():
    from pam_b200 import fused
    dev = torch.device("cuda", 0)
    qkv = torch.randn(2, 9, 3 * 8, device=dev)
    assert not fused.attention_supported(qkv, 4, False)             # exact backward: chain of operators
    assert not fused.attention_supported(qkv, 4, (True, False))
    assert not fused.attention_supported(qkv, 5, True)              # 24 is not 3 * 5 * head_dim
    assert not fused.attention_supported(qkv.cpu(), 4, True)


def heads_chain(ops, q, k, v, heads, mask, kw):
    """The explicit branch of the fairseq fork's attention after the projections
    (fairseq/modules/multihead_attention.py:618-783): heads split into copies, bmm, mask, softmax, bmm."""
    B, T, d = q.shape
    S, hd = k.shape[1], d // heads
    split = lambda t, L: t.reshape(B, L, heads, hd).transpose(1, 2).reshape(B * heads, L, hd)
    w = ops.bmm(split(q, T), split(k, S).transpose(1, 2), **kw)
    if mask is not None:
        w = w + mask
    w = ops.softmax(w, dim=-1, **kw)
    return ops.bmm(w, split(v, S), **kw).reshape(B, heads, T, hd).transpose(1, 2).reshape(B, T, d)


@pytest.mark.parametrize("B,T,S,heads,hd,masked", [(128, 32, 32, 4, 128, True), (128, 32, 32, 4, 128, False), (3, 17, 29, 4, 16, False),
                                                    (2, 40, 40, 8, 8, True), (5, 1, 7, 2, 4, False), (2, 200, 197, 3, 64, False)])
@pytest.mark.parametrize("offset", [None, 1.0552])
def test_strided_attention_over_separate_projections_equals_the_chain(B, T, S, heads, hd, masked, offset):
    import pam_b200 as pam
    from pam_b200 import fused
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(B * 100 + T + S)
    d = heads * hd
    q0, k0, v0 = (torch.randn(B, L, d, generator=g).to(dev) for L in (T, S, S))
    dout = torch.randn(B, T, d, generator=g).to(dev)
    mask = torch.triu(torch.full((T, S), float("-inf")), diagonal=1).to(dev) if masked else None
    kw = dict(KW, offset=offset)
    assert fused.attention_heads_supported(q0, k0, v0, heads, mask, True)
    grads = []
    for use_fused in (True, False):
        q, k, v = (t.clone().requires_grad_() for t in (q0, k0, v0))
        y = fused.attention_heads(q, k, v, heads, mask, offset=offset) if use_fused else heads_chain(pam, q, k, v, heads, mask, kw)
        y.backward(dout)
        grads.append((y.detach(), q.grad, k.grad, v.grad))
    for name, a, b in zip(("context", "d q", "d k", "d v"), *grads):
        assert_bits_equal(a, b, name)
