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
