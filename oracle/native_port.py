"""TEST INFRASTRUCTURE / CPU BASELINE — a port of the reference's "native" PyTorch path
(epfml/pam pam/native.py), the float-log formulation that is the reference's only CPU
implementation: pam(a, b) = sign * 2^floor(s) * (1 + s - floor(s)) with s = log2'(|a|) + log2'(|b|)
and log2'(x) = floor(log2 x) + mantissa fraction.

It exists so that the benchmark can time the reference's CPU arithmetic on a machine where the
reference tree is not mounted; it is never imported by the shipped package.  Its results are NOT
bit-identical to the kernels' integer arithmetic (they agree to ~1e-6 relative; the reference's
own tests only ask for allclose).  Checked against values produced by the real pam/native.py in
tests/golden/pam_golden.npz (keys native/*).
"""
import torch


def _log2_pa(x):
    # native.py:11-32: exponent + mantissa fraction of |x|; -inf exponent and 0 fraction for 0
    x = x.abs()
    e = torch.floor(torch.log2(x))
    p = torch.exp2(e)
    return e + (x - p) / torch.where(p > 0, p, torch.ones_like(p))


def _exp2_pa(s):
    # native.py:35-41
    f = torch.floor(s)
    return torch.exp2(f) * torch.where(f.isfinite(), 1 + s - f, torch.ones_like(s))


def pam(a, b, offset=None):
    # native.py:44-64
    out = torch.sign(a) * torch.sign(b) * _exp2_pa(_log2_pa(a) + _log2_pa(b))
    if offset is not None:
        out = pam(out, torch.full_like(out, offset))
    return out


def pad(a, b, offset=None):
    # native.py:150-169
    out = torch.sign(a) / torch.sign(b) * _exp2_pa(_log2_pa(a) - _log2_pa(b))
    if offset is not None:
        out = pad(out, torch.full_like(out, offset))
    return out


def matmul(A, B, offset=None, row_chunk=None):
    """native.py:117-131: broadcast to [n, k, m], PAM elementwise, sum over k.  The reference
    materialises the whole n*k*m tensor; rows are independent, so it is evaluated in row chunks
    sized to ~256 MB of temporaries (identical results, bounded memory)."""
    n, k = A.shape
    m = B.shape[1]
    if row_chunk is None:
        row_chunk = max(1, min(n, (64 << 20) // max(1, k * m)))
    out = torch.empty(n, m, dtype=A.dtype)
    Bv = B.view(1, k, m)
    for r in range(0, n, row_chunk):
        out[r:r + row_chunk] = torch.sum(pam(A[r:r + row_chunk].reshape(-1, k, 1), Bv, offset), dim=1)
    return out


def matmul_approx_bwd(A, B, G, offset=None):
    """Gradients of the approx_bwd matmul (native.py:96-107 via broadcasting): dA = G (x) B^T,
    dB = A^T (x) G with PAM products."""
    return matmul(G, B.T, offset), matmul(A.T, G, offset)


def layer_norm(x, weight, bias, eps, offset=None):
    """pam_ops.layer_norm (pam/pam_ops.py:350-378) over the native primitives, forward only."""
    n = torch.tensor(float(x.shape[-1]))
    mu = pad(x.sum(-1, keepdim=True), n.expand(x.shape[0], 1), offset)
    c = x - mu
    var = pad(pam(c, c, offset).sum(-1, keepdim=True), n.expand(x.shape[0], 1), offset)
    v = var + eps
    half = torch.full_like(v, 0.5)
    # pow(v, 0.5) = exp2(pam(log2(v), 0.5)); exp2 / log2 of the op library wrap a PAM by 1.0
    denom = torch.where(v == 0, torch.zeros_like(v), _exp2_pa(pam(_log2_pa(v), half, offset)))
    out = pad(c, denom.expand_as(c), offset)
    if weight is not None:
        out = pam(out, weight.expand_as(out), offset)
    return out if bias is None else out + bias
