"""Test infrastructure: the fused pam_ln kernel's arithmetic replayed on the CPU with the oracle's
scalar functions, with pluggable summation orders.

With torch.sum as the summation this chain reproduces the reference's layer_norm forward and
backward bit for bit (checked against the fixtures generated from the reference); with the
kernel's own order (per-lane running sums joined by a butterfly over the 32 lanes, rows joined
per warp / CTA / grid) it predicts the CUDA kernel's output bit for bit.  Together the two give a
bit-exact chain from the reference to the kernel although their sums associate differently."""
import math

import torch

from oracle import pam_oracle


def _f(v):
    return torch.tensor(v, dtype=torch.float32)


class Chain:
    def __init__(self, offset, rowsum, colsum):
        self.K = pam_oracle.kernels()
        self.off = 1.0 if offset is None else offset
        self.rowsum, self.colsum = rowsum, colsum

    def _b(self, *ts):
        return [t.contiguous() for t in torch.broadcast_tensors(*ts)]

    def mul(self, a, b, off=None):
        return self.K.pam_fwd(*self._b(a, b), self.off if off is None else off)

    def div(self, a, b):
        return self.K.pad_fwd(*self._b(a, b), self.off)

    def mul_bwd(self, a, b, dc, off=None):
        return self.K.pam_bwd(*self._b(a, b, dc), self.off if off is None else off)

    def div_bwd(self, a, b, dc):
        return self.K.pad_bwd(*self._b(a, b, dc), self.off)

    def run(self, x, w, b, g, eps, approx):
        K, off = self.K, self.off
        n = x.shape[-1]
        nf, one, half, ln2 = _f(float(n)), _f(1.0), _f(0.5), _f(math.log(2.0))
        x, g = x.reshape(-1, n), g.reshape(-1, n)
        s1 = self.rowsum(x)
        c = x - self.div(s1, nf)
        s2 = self.rowsum(self.mul(c, c))
        v = self.div(s2, nf) + _f(eps)
        l = K.pa_log_fwd(v, 2.0, off)
        m = self.mul(l, half)
        e = K.pa_exp_fwd(m, 2.0, off)
        denom = torch.where(v == 0, torch.zeros_like(e), e)
        xn = self.div(c, denom)
        y = xn if w is None else self.mul(xn, w)
        if b is not None:
            y = y + b
        recip, recip_n = self.div(one, denom), self.div(one, nf)
        dw = db = None
        dxn = g
        if w is not None:
            dw = self.colsum(self.mul(g, xn) if approx else self.mul_bwd(w, xn, g))
            db = self.colsum(g)
            dxn = self.mul(g, w) if approx else self.mul_bwd(xn, w, g)
        dden = -self.mul(self.div(xn, denom), dxn) if approx else self.div_bwd(c, denom, dxn)
        dc = self.mul(recip, dxn) if approx else self.mul_bwd(c, recip, dxn, 1.0)
        d_denom = self.rowsum(dden)
        d_e = torch.where(v == 0, torch.zeros_like(d_denom), d_denom)
        d_m = self.mul(self.mul(e, ln2), d_e) if approx else K.pa_exp_bwd(m, d_e, 2.0, off)
        d_l = self.mul(d_m, half) if approx else self.mul_bwd(l, half, d_m)
        d_v = self.div(self.div(d_l, v), ln2) if approx else K.pa_log_bwd(v, d_l, 2.0, off)
        d_s2 = self.mul(recip_n, d_v) if approx else self.mul_bwd(s2, recip_n, d_v, 1.0)
        dsq = self.mul(d_s2, c) if approx else self.mul_bwd(c, c, d_s2)
        dc = (dc + dsq) + dsq
        d_mu = -self.rowsum(dc)
        d_s1 = self.mul(recip_n, d_mu) if approx else self.mul_bwd(s1, recip_n, d_mu, 1.0)
        return y, dc + d_s1, dw, db


def torch_rowsum(t):
    return t.sum(-1, keepdim=True)


def torch_colsum(t):
    return t.sum(0)


def kernel_rowsum(vec):
    """Summation order of the kernel: lane L holds the columns (q*32 + L)*vec + j in the order
    (q, j), adds them one by one starting from +0, then the 32 lane sums are joined by a
    butterfly (xor 16, 8, 4, 2, 1)."""
    def rowsum(t):
        rows, n = t.shape
        chunks = -(-n // (32 * vec))
        padded = torch.zeros(rows, chunks * 32 * vec)
        padded[:, :n] = t
        lanes = padded.view(rows, chunks, 32, vec).permute(0, 2, 1, 3).reshape(rows, 32, chunks * vec)
        part = torch.zeros(rows, 32)
        for i in range(chunks * vec):
            part = part + lanes[:, :, i]
        idx = torch.arange(32)
        for d in (16, 8, 4, 2, 1):
            part = part + part[:, idx ^ d]
        return part[:, :1].contiguous()
    return rowsum


def kernel_colsum(rows_total, grid, warps_per_cta=4, grad_warps=8):
    """Order of the dweight / dbias sums in the kernel: warp w of CTA c adds its rows
    (c*4 + w, + grid*4, ...) in order from +0; the four warps of a CTA are added in order; the
    second kernel's warp j adds the CTA sums j, j + 8, ... in order from +0 and the eight warp
    sums are added in order."""
    def colsum(t):
        rows, n = t.shape
        nwarps = grid * warps_per_cta
        warp_sums = torch.zeros(nwarps, n)
        for r in range(rows):
            warp_sums[r % nwarps] = warp_sums[r % nwarps] + t[r]
        ws = warp_sums.view(grid, warps_per_cta, n)
        cta = ws[:, 0]
        for wdx in range(1, warps_per_cta):
            cta = cta + ws[:, wdx]
        subs = torch.zeros(grad_warps, n)
        for k in range(grid):
            subs[k % grad_warps] = subs[k % grad_warps] + cta[k]
        total = subs[0]
        for j in range(1, grad_warps):
            total = total + subs[j]
        return total
    return colsum
