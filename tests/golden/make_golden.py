"""Generates tests/golden/pam_golden.npz from the reference itself (run where the reference tree
is mounted; the fixture file is committed, this script documents how it was made).

    python tests/golden/make_golden.py

How the reference is run without a GPU: the reference's Python (pam/pam_ops.py,
pam/cuda_bindings.py, pam/pam_opt.py, pam/native.py) is imported unmodified.  Its import-time JIT
build (cuda_bindings.py:17-25) is replaced by a stand-in for the compiled module whose 14
functions evaluate the reference's OWN scalar device functions (pam/cuda_kernels.cu:15-136,
compiled for the host as oracle/_ref/libpam_ref.so) over CPU tensors.  pam_ops dispatches on
``tensor.is_cuda``; pointing its ``native`` name at ``cuda_bindings`` makes CPU tensors take the
kernel path, so every value below is produced by the reference's autograd functions and op
library over the reference's integer arithmetic.  The ``native/*`` entries use the untouched
float-log path (pam/native.py) instead.

The Adam entries replay submodules/fairseq/fairseq/optim/adam.py:226-252 with the reference's
``pam.mul/div/pow`` (fairseq itself cannot be imported here: omegaconf and friends are absent).
"""
import math
import os
import pathlib
import sys

import numpy as np
import torch

ROOT = pathlib.Path(__file__).resolve().parents[2]
REF = pathlib.Path(os.environ.get("PAM_REFERENCE_ROOT", "/root/reference"))
sys.path.insert(0, str(ROOT))

from oracle import build as oracle_build  # noqa: E402
from oracle import pam_oracle  # noqa: E402

oracle_build.build_oracle()
assert oracle_build.build_ref() is not None, "reference tree not mounted"

import torch.utils.cpp_extension as cpp_ext  # noqa: E402

cpp_ext.load = lambda **kw: pam_oracle.CpuKernels("reference")
sys.path.insert(0, str(REF))
import pam  # noqa: E402  (the reference package)
from pam import cuda_bindings, native, pam_ops  # noqa: E402

real_native = native
pam_ops.native = cuda_bindings  # CPU tensors -> kernel path

OUT = {}
g = torch.Generator().manual_seed(20261125)


def put(name, t):
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu().numpy()
    OUT[name] = np.ascontiguousarray(t)


def randn(*shape):
    return torch.randn(*shape, generator=g)


SPECIALS = [0.0, -0.0, 1e-40, -1e-40, 1.4e-45, -1.4e-45, 1e30, -1e30, 1e-30, -1e-30,
            float("inf"), float("-inf"), float("nan"), 3e38, 1.2e-38, 1.0, -1.0, 2.0, 0.5]


def with_specials(t, every=7):
    t = t.clone().view(-1)
    idx = torch.arange(0, t.numel(), every)
    t[idx] = torch.tensor(SPECIALS, dtype=torch.float32)[torch.arange(idx.numel()) % len(SPECIALS)]
    return t


def grads(fn, *inputs, gout=None):
    leaves = [t.clone().requires_grad_() for t in inputs]
    out = fn(*leaves)
    if gout is None:
        gout = torch.ones_like(out)
    out.backward(gout)
    return out.detach(), [leaf.grad for leaf in leaves]


# ---- elementwise mul / div, all four (offset, approx) combinations -------------------------------
n = 3000
a = with_specials(randn(n) * torch.exp2(torch.randint(-30, 30, (n,), generator=g).float()), 7)
b = with_specials(randn(n) * torch.exp2(torch.randint(-30, 30, (n,), generator=g).float()), 11)
dc = with_specials(randn(n), 13)
put("ew/a", a), put("ew/b", b), put("ew/dc", dc)
for oname, off in (("none", None), ("o1", 1.0552)):
    for approx in (False, True):
        tag = f"{oname}/{'approx' if approx else 'exact'}"
        for opname, op in (("mul", pam_ops.mul), ("div", pam_ops.div)):
            y, (da, db) = grads(lambda x, z: op(x, z, offset=off, approx_bwd=approx), a, b, gout=dc)
            put(f"ew/{opname}/{tag}/y", y), put(f"ew/{opname}/{tag}/da", da), put(f"ew/{opname}/{tag}/db", db)

# broadcasting + scalar operands (row vector, column vector, python scalar)
m2 = randn(9, 13)
rowv, colv = randn(13), randn(9, 1)
put("bc/m", m2), put("bc/row", rowv), put("bc/col", colv)
for opname, op in (("mul", pam_ops.mul), ("div", pam_ops.div)):
    y, (d0, d1) = grads(lambda x, z: op(x, z, approx_bwd=True), m2, rowv)
    put(f"bc/{opname}/row/y", y), put(f"bc/{opname}/row/d0", d0), put(f"bc/{opname}/row/d1", d1)
    y, (d0, d1) = grads(lambda x, z: op(x, z, approx_bwd=False), m2, colv)
    put(f"bc/{opname}/col/y", y), put(f"bc/{opname}/col/d0", d0), put(f"bc/{opname}/col/d1", d1)
    y, (d0,) = grads(lambda x: op(x, 0.3, approx_bwd=True), m2)
    put(f"bc/{opname}/scalar/y", y), put(f"bc/{opname}/scalar/d0", d0)
put("bc/scalar_scalar", np.array([pam_ops.mul(1.3, -1.3), pam_ops.div(0.1, 9999.0), pam_ops.pow(2.5, 0.5)],
                                  dtype=np.float64))

# ---- exp / log -----------------------------------------------------------------------------------
x = with_specials(randn(n) * 20, 17)
xp = with_specials(randn(n).abs() * torch.exp2(torch.randint(-30, 30, (n,), generator=g).float()), 19)
put("el/x", x), put("el/xp", xp)
for bname, base in (("e", math.e), ("2", 2.0), ("10", 10.0)):
    for oname, off in (("none", None), ("o1", 1.0552)):
        for approx in (False, True):
            tag = f"{bname}/{oname}/{'approx' if approx else 'exact'}"
            y, (dx,) = grads(lambda t: pam_ops.exp(t, base, offset=off, approx_bwd=approx), x, gout=dc)
            put(f"el/exp/{tag}/y", y), put(f"el/exp/{tag}/dx", dx)
            y, (dx,) = grads(lambda t: pam_ops.log(t, base, offset=off, approx_bwd=approx), xp, gout=dc)
            put(f"el/log/{tag}/y", y), put(f"el/log/{tag}/dx", dx)
pw_a = with_specials(randn(500).abs(), 23)
pw_a[5] = 0.0
put("pow/a", pw_a)
for approx in (False, True):
    y, (dx,) = grads(lambda t: pam_ops.pow(t, 0.5, approx_bwd=approx), pw_a)
    put(f"pow/{'approx' if approx else 'exact'}/y", y), put(f"pow/{'approx' if approx else 'exact'}/dx", dx)

# ---- matmul: the reference's own test matrices (pam/test_pam.py:96-97,129-130) and random ones ----
for tag, shift in (("ref21", 2.1), ("ref20", 2.0)):
    A = (torch.arange(20) ** 3 % 7 - shift).reshape(5, 4).float()
    B = (torch.arange(12) ** 2 % 5 - shift).reshape(3, 4).float().T
    gC = torch.arange(15).float().reshape(5, 3)
    put(f"mm/{tag}/A", A), put(f"mm/{tag}/B", B.contiguous()), put(f"mm/{tag}/gC", gC)
    for approx in (False, True):
        y, (dA, dB) = grads(lambda p, q: pam_ops.matmul(p, q, approx_bwd=approx), A, B, gout=gC)
        k = "approx" if approx else "exact"
        put(f"mm/{tag}/{k}/y", y), put(f"mm/{tag}/{k}/dA", dA), put(f"mm/{tag}/{k}/dB", dB)

A = with_specials(randn(33, 70), 29).view(33, 70)
B = with_specials(randn(70, 45), 31).view(70, 45)
gC = randn(33, 45)
put("mm/rand/A", A), put("mm/rand/B", B), put("mm/rand/gC", gC)
for oname, off in (("none", None), ("o1", 1.0552)):
    for approx in (False, True):
        k = f"{oname}/{'approx' if approx else 'exact'}"
        y, (dA, dB) = grads(lambda p, q: pam_ops.matmul(p, q, offset=off, approx_bwd=approx), A, B, gout=gC)
        put(f"mm/rand/{k}/y", y), put(f"mm/rand/{k}/dA", dA), put(f"mm/rand/{k}/dB", dB)
put("mm/rand/standard/y", cuda_bindings.standard_matmul(A.nan_to_num(0, 0, 0), B.nan_to_num(0, 0, 0)))

A3, B3, g3 = randn(3, 17, 33), randn(3, 33, 9), randn(3, 17, 9)
put("bmm/A", A3), put("bmm/B", B3), put("bmm/gC", g3)
for approx in (False, True):
    k = "approx" if approx else "exact"
    y, (dA, dB) = grads(lambda p, q: cuda_bindings.pam_bmm(p, q, approx_bwd=approx), A3, B3, gout=g3)
    put(f"bmm/{k}/y", y), put(f"bmm/{k}/dA", dA), put(f"bmm/{k}/dB", dB)

# ---- Linear module (pam_ops.py:259-285) ------------------------------------------------------------
lin = pam.Linear(24, 10, approx_bwd=True)
X = randn(4, 6, 24)
put("linear/X", X), put("linear/W", lin.weight), put("linear/b", lin.bias)
Xl = X.clone().requires_grad_()
yl = lin(Xl)
gl = randn(*yl.shape)
yl.backward(gl)
put("linear/gy", gl), put("linear/y", yl), put("linear/dX", Xl.grad)
put("linear/dW", lin.weight.grad), put("linear/db", lin.bias.grad)

# ---- reductions and normalisation ------------------------------------------------------------------
S = randn(6, 5, 11) * 3
S_masked = S.clone()
S_masked[:, :, -3:] = float("-inf")
gS = randn(6, 5, 11)
put("sm/x", S), put("sm/x_masked", S_masked), put("sm/g", gS)
for oname, off in (("none", None), ("o1", 1.0552)):
    for approx in (False, True):
        k = f"{oname}/{'approx' if approx else 'exact'}"
        kw = dict(offset=off, approx_bwd=approx)
        y, (dx,) = grads(lambda t: pam_ops.softmax(t, dim=-1, **kw), S, gout=gS)
        put(f"sm/softmax/{k}/y", y), put(f"sm/softmax/{k}/dx", dx)
        y, (dx,) = grads(lambda t: pam_ops.softmax(t, dim=-1, **kw), S_masked, gout=gS)
        put(f"sm/softmax_masked/{k}/y", y), put(f"sm/softmax_masked/{k}/dx", dx)
        y, (dx,) = grads(lambda t: pam_ops.softmax(t, dim=1, **kw), S, gout=gS)
        put(f"sm/softmax_dim1/{k}/y", y), put(f"sm/softmax_dim1/{k}/dx", dx)
        y, (dx,) = grads(lambda t: pam_ops.log_softmax(t, dim=-1, **kw), S, gout=gS)
        put(f"sm/log_softmax/{k}/y", y), put(f"sm/log_softmax/{k}/dx", dx)
        y, (dx,) = grads(lambda t: pam_ops.logsumexp(t, dim=-1, **kw), S, gout=gS[..., 0])
        put(f"sm/logsumexp/{k}/y", y), put(f"sm/logsumexp/{k}/dx", dx)
        y, (dx,) = grads(lambda t: pam_ops.mean(t, dim=-1, keepdim=True, **kw), S, gout=gS[..., :1])
        put(f"sm/mean/{k}/y", y), put(f"sm/mean/{k}/dx", dx)

Xn = randn(7, 3, 48) * 2 + 0.5
Xn[2, 1] = 0.25            # a constant row: variance 0 -> pow(eps)
wn, bn, gn = randn(48).abs() + 0.5, randn(48), randn(7, 3, 48)
put("ln/x", Xn), put("ln/w", wn), put("ln/b", bn), put("ln/g", gn)
for oname, off in (("none", None), ("o1", 1.0552)):
    for approx in (False, True):
        k = f"{oname}/{'approx' if approx else 'exact'}"
        kw = dict(offset=off, approx_bwd=approx)
        y, (dx, dw, db) = grads(lambda t, w_, b_: pam_ops.layer_norm(t, 48, w_, b_, 1e-5, **kw), Xn, wn, bn, gout=gn)
        put(f"ln/affine/{k}/y", y), put(f"ln/affine/{k}/dx", dx), put(f"ln/affine/{k}/dw", dw), put(f"ln/affine/{k}/db", db)
        y, (dx,) = grads(lambda t: pam_ops.layer_norm(t, (48,), None, None, 1e-6, **kw), Xn, gout=gn)
        put(f"ln/plain/{k}/y", y), put(f"ln/plain/{k}/dx", dx)

# ---- cross entropy backward (pam_opt.py:6-62) --------------------------------------------------------
from shared.modules import factories  # noqa: E402

op_dict = factories.get_function_dict('{"type": "pam", "dkwargs": {"approx_bwd": true}}')
logits, target = randn(12, 9) * 2, torch.randint(0, 9, (12,), generator=g)
target[3] = 1
put("ce/x", logits), put("ce/t", target.numpy().astype(np.int64))
for ls in (0.0, 0.1):
    y, (dx,) = grads(lambda t: pam.cross_entropy(t, target, None, 1, "mean", ls, op_dict=op_dict), logits)
    put(f"ce/ls{ls}/y", y), put(f"ce/ls{ls}/dx", dx)

# ---- PAM Adam (fairseq/optim/adam.py:226-252), three steps ----------------------------------------------
p = randn(257)
m, v = torch.zeros_like(p), torch.zeros_like(p)
lr, betas, eps, wd = 5e-4, (0.9, 0.98), 1e-8, 1e-4
put("adam/p0", p)
ops = factories.get_function_dict("pam")
for step in (1, 2, 3):
    grad = with_specials(randn(257) * 0.1, 41) if step == 2 else randn(257) * 0.1
    grad = grad.nan_to_num(0.0, 0.0, 0.0)
    put(f"adam/g{step}", grad)
    b1, b2 = betas
    m = ops["mul"](m, b1) + ops["mul"](grad, 1 - b1)
    v = ops["mul"](v, b2)
    v = v + ops["mul"](ops["mul"](grad, grad), 1 - b2)
    denom = ops["pow"](v, 0.5) + eps
    step_size = lr * math.sqrt(1 - b2 ** step) / (1 - b1 ** step)
    p = p - ops["mul"](p, wd * lr)
    p = p - ops["mul"](ops["div"](m, denom), step_size)
    put(f"adam/p{step}", p), put(f"adam/m{step}", m), put(f"adam/v{step}", v)

# ---- the untouched float-log "native" path (pam/native.py), used to check the timed CPU port ----------
na, nb = randn(2000), randn(2000) * 0.02
put("native/a", na), put("native/b", nb)
put("native/pam", real_native.pam_fwd(na, nb))
put("native/pam_off", real_native.pam_fwd(na, nb, offset=1.0552))
put("native/pad", real_native.pad_fwd(na, nb))
nA, nB, nG = randn(20, 31), randn(31, 17), randn(20, 17)
put("native/A", nA), put("native/B", nB), put("native/G", nG)
y, (dA, dB) = grads(lambda p_, q_: real_native.pam_matmul(p_, q_, approx_bwd=True), nA, nB, gout=nG)
put("native/mm/y", y), put("native/mm/dA", dA), put("native/mm/dB", dB)
pam_ops.native = real_native
y, (dx,) = grads(lambda t: pam_ops.layer_norm(t, 48, wn, bn, 1e-5, approx_bwd=True, use_kernel=False), Xn, gout=gn)
put("native/ln/y", y), put("native/ln/dx", dx)

path = pathlib.Path(__file__).with_name("pam_golden.npz")
np.savez_compressed(path, **OUT)
print(f"{len(OUT)} arrays -> {path} ({path.stat().st_size / 1024:.0f} KiB)")
