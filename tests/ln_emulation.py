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


    # ---- softmax / logsumexp over the last dimension (pam_b200/csrc/softmax.cu) -------------------
    def _scaled(self, x):
        log2e = _f(math.log2(math.e))
        masked = x == float("-inf")
        scaled = torch.where(masked, torch.full_like(x, float("-inf")), self.mul(x, log2e))
        return masked, scaled, torch.floor(torch.max(scaled)), log2e

    def softmax(self, x, g, approx):
        K, off = self.K, self.off
        n = x.shape[-1]
        x, g = x.reshape(-1, n), g.reshape(-1, n)
        ln2, one = _f(math.log(2.0)), _f(1.0)
        masked, scaled, shift, log2e = self._scaled(x)
        adj = scaled - shift
        big = K.pa_exp_fwd(adj, 2.0, off)
        e = torch.where(masked, torch.zeros_like(big), big)
        total = self.rowsum(e)
        y = self.div(e, total)
        recip = self.div(one, total)
        dden = -self.mul(self.div(self.div(e, total), total), g) if approx else self.div_bwd(e, total, g)
        de = self.mul(recip, g) if approx else self.mul_bwd(e, recip, g, 1.0)
        d_big = torch.where(masked, torch.zeros_like(de), de + self.rowsum(dden))
        d_adj = self.mul(self.mul(e, ln2), d_big) if approx else K.pa_exp_bwd(adj, d_big, 2.0, off)
        d_s = torch.where(masked, torch.zeros_like(d_adj), d_adj)
        dx = self.mul(d_s, log2e) if approx else self.mul_bwd(x, log2e, d_s)
        return y, dx

    def logsumexp(self, x, g, approx):
        """x [rows, n], g [rows]; the log2 of the row sum always runs with offset 1 and the exact
        backward (pam_ops.py:341)."""
        K, off = self.K, self.off
        n = x.shape[-1]
        x, g = x.reshape(-1, n), g.reshape(-1, 1)
        ln2, one = _f(math.log(2.0)), _f(1.0)
        _, scaled, shift, log2e = self._scaled(x)
        adj = scaled - shift
        e = K.pa_exp_fwd(adj, 2.0, off)
        total = self.rowsum(e)
        u = shift + K.pa_log_fwd(total, 2.0, 1.0)
        y = self.div(u, log2e)
        recip = self.div(one, log2e)
        d_u = self.mul(recip, g) if approx else self.mul_bwd(u, recip, g, 1.0)
        d_total = K.pa_log_bwd(total, d_u, 2.0, 1.0)
        d_adj = self.mul(self.mul(e, ln2), d_total) if approx else K.pa_exp_bwd(adj, d_total.expand_as(adj).contiguous(), 2.0, off)
        dx = self.mul(d_adj, log2e) if approx else self.mul_bwd(x, log2e, d_adj)
        return y.reshape(-1), dx


def torch_rowsum(t):
    return t.sum(-1, keepdim=True)


def torch_colsum(t):
    return t.sum(0)


def kernel_rowsum(vec, warps=1):
    """Summation order of the row kernels: thread t of a group of warps*32 holds the columns
    (q*group + t)*vec + j in the order (q, j) and adds them one by one starting from +0; the 32
    lane sums of each warp are joined by a butterfly (xor 16, 8, 4, 2, 1); the warp sums, if there
    is more than one warp, are added in warp order."""
    group = 32 * warps

    def rowsum(t):
        rows, n = t.shape
        chunks = -(-n // (group * vec))
        padded = torch.zeros(rows, chunks * group * vec)
        padded[:, :n] = t
        lanes = padded.view(rows, chunks, group, vec).permute(0, 2, 1, 3).reshape(rows, group, chunks * vec)
        part = torch.zeros(rows, group)
        for i in range(chunks * vec):
            part = part + lanes[:, :, i]
        part = part.view(rows, warps, 32)
        idx = torch.arange(32)
        for d in (16, 8, 4, 2, 1):
            part = part + part[:, :, idx ^ d]
        total = part[:, 0, 0]
        for wdx in range(1, warps):
            total = total + part[:, wdx, 0]
        return total.reshape(rows, 1).contiguous()
    return rowsum


def kernel_colsum(rows_total, grid, warps_per_cta=4, grad_warps=32, rows_per_warp=1):
    """Order of the dweight / dbias sums in the kernel: a warp takes `rows_per_warp` consecutive
    rows per pass (groups g = warp, warp + grid*4, ...) and adds its rows in order from +0; the four
    warps of a CTA are added in order; the second kernel's warp j adds the CTA sums j, j + 32, ...
    in order from +0 and the 32 warp sums are added in order."""
    def colsum(t):
        rows, n = t.shape
        nwarps = grid * warps_per_cta
        warp_sums = torch.zeros(nwarps, n)
        for r in range(rows):
            owner = (r // rows_per_warp) % nwarps
            warp_sums[owner] = warp_sums[owner] + t[r]
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
