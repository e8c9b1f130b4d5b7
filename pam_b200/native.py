"""Names of the reference's ``pam/native.py``, served by the CUDA kernels.

In the reference this module is a second, pure-PyTorch implementation (float ``log2/floor/exp2``)
that also runs on CPU and whose results differ from its kernels' in the last bits.  This package
has a single arithmetic — the integer formulation of the kernels — so the same names are kept
for callers and tests that import them, and they compute with the kernels.  CPU tensors raise.
"""
import math

import torch

from . import cuda_bindings
from .cuda_bindings import cuda_kernels, _offset


def get_exp_mantissa(x):
    """floor(log2|x|) and the mantissa fraction in [0, 1) of each element (native.py:11-21);
    exact bit extraction, -inf / 0 for zeros."""
    frac, expo = torch.frexp(x.abs())
    x_e = torch.where(x == 0, float("-inf"), (expo - 1).to(x.dtype))
    return x_e, torch.where(x == 0, 0.0, frac * 2 - 1)


def pa_log2_fwd(x):
    return cuda_kernels.pa_log_fwd(x.abs(), 2.0, 1.0)


def pa_exp2_fwd(x):
    return cuda_kernels.pa_exp_fwd(x, 2.0, 1.0)


def pam_fwd(A, B, *, offset=None):
    """Differentiable PAM product with the exact backward (what autograd derives from the
    reference's float formulation, native.py:41-60)."""
    return cuda_bindings.pam(A, B, offset=offset, approx_bwd=False)


@torch.no_grad()
def pam_bwd(A, B, delta_C, *, offset=None):
    return cuda_kernels.pam_bwd(A, B, delta_C, _offset(offset))


pam = cuda_bindings.pam
pam_matmul = cuda_bindings.pam_matmul


def pam_matmul_fwd(A, B, *, offset=None):
    return cuda_bindings.pam_matmul(A, B, offset=offset, approx_bwd=False)


def pad_fwd(A, B, *, offset=None):
    return cuda_bindings.pad(A, B, offset=offset, approx_bwd=False)


pad = cuda_bindings.pad


def pa_exp_fwd(x, base=math.e, offset=None):
    return cuda_bindings.pa_exp(x, base=base, offset=offset, approx_bwd=False)


def pa_log_fwd(x, base=math.e, offset=None):
    return cuda_bindings.pa_log(x, base=base, offset=offset, approx_bwd=False)


pa_exp = cuda_bindings.pa_exp
pa_exp2 = cuda_bindings.pa_exp2
pa_log = cuda_bindings.pa_log
pa_log2 = cuda_bindings.pa_log2
