"""The PAM operator library — functions and modules with the names, arguments and semantics of
the reference's ``pam/pam_ops.py``, computed by the sm_100a kernels of this package.

Every function takes the reference's keyword-only ``offset``, ``approx_bwd`` and ``use_kernel``.
``use_kernel`` is accepted for compatibility and ignored: there is no non-kernel path here, and a
CPU tensor raises instead of silently taking a slow route.  Python numbers are passed to the
kernels by value (the reference first copies each one into a 0-d device tensor).
"""
import math

import torch

from . import cuda_bindings, fused, utils
from .utils import is_number

__all__ = [
    "mul", "div", "exp", "exp2", "log", "log2", "pow", "matmul", "bmm", "linear", "conv2d", "conv2d_group",
    "Conv2d", "Linear", "mean", "softmax", "logsumexp", "log_softmax", "layer_norm", "LayerNorm",
]


def _scalar_device():
    if not torch.cuda.is_available():
        raise RuntimeError("pam_b200 needs a CUDA device even for Python-number operands (no CPU path)")
    return torch.device("cuda", torch.cuda.current_device())


def _lift(*values):
    """If every operand is a Python number, the first becomes a 0-d CUDA tensor so that a kernel
    can evaluate the call; the result is turned back into a float by ``utils.demote_tensor``."""
    if all(is_number(v) for v in values):
        first = torch.tensor(float(values[0]), dtype=torch.float32, device=_scalar_device())
        return (first, *values[1:])
    return values


def mul(A, B, *, offset=None, approx_bwd=False, use_kernel=True):
    # pam/pam_ops.py:16-22
    tA, tB = _lift(A, B)
    return utils.demote_tensor(cuda_bindings.pam(tA, tB, offset=offset, approx_bwd=approx_bwd), (A, B))


def div(A, B, *, offset=None, approx_bwd=False, use_kernel=True):
    # pam/pam_ops.py:25-31
    tA, tB = _lift(A, B)
    return utils.demote_tensor(cuda_bindings.pad(tA, tB, offset=offset, approx_bwd=approx_bwd), (A, B))


def exp(A, base=math.e, *, offset=None, approx_bwd=False, use_kernel=True):
    (tA,) = _lift(A)
    return utils.demote_tensor(cuda_bindings.pa_exp(tA, base=base, offset=offset, approx_bwd=approx_bwd), (A,))


def exp2(A, *, offset=None, approx_bwd=False, use_kernel=True):
    (tA,) = _lift(A)
    return utils.demote_tensor(cuda_bindings.pa_exp2(tA, offset=offset, approx_bwd=approx_bwd), (A,))


def log(A, base=math.e, *, offset=None, approx_bwd=False, use_kernel=True):
    (tA,) = _lift(A)
    return utils.demote_tensor(cuda_bindings.pa_log(tA, base=base, offset=offset, approx_bwd=approx_bwd), (A,))


def log2(A, *, offset=None, approx_bwd=False, use_kernel=True):
    (tA,) = _lift(A)
    return utils.demote_tensor(cuda_bindings.pa_log2(tA, offset=offset, approx_bwd=approx_bwd), (A,))


def pow(A, B, *, offset=None, approx_bwd=False, use_kernel=True):
    """A**B as exp2(B * log2(A)) in PAM arithmetic, with 0**B = 0 (pam/pam_ops.py:70-79)."""
    kw = dict(offset=offset, approx_bwd=approx_bwd)
    tA = _lift(A)[0] if is_number(A) else A
    out = torch.where(tA == 0, 0, exp2(mul(log2(tA, **kw), B, **kw), **kw))
    return utils.demote_tensor(out, (A, B))


def matmul(A, B, *, offset=None, approx_bwd=False, use_kernel=True):
    return cuda_bindings.pam_matmul(A, B, offset=offset, approx_bwd=approx_bwd)


def bmm(A, B, *, offset=None, approx_bwd=False, use_kernel=True):
    assert A.dim() == B.dim() == 3
    assert A.shape[0] == B.shape[0]
    assert A.shape[2] == B.shape[1]
    return cuda_bindings.pam_bmm(A, B, offset=offset, approx_bwd=approx_bwd)


def linear(X, W, bias=None, *, offset=None, approx_bwd=False, use_kernel=True):
    """X @ W.T (+ bias with an ordinary add) over the flattened leading dimensions
    (pam/pam_ops.py:107-115).  W is [out, in]: both operands are contiguous along K."""
    lead = X.shape[:-1]
    X2 = X.reshape(-1, X.shape[-1])
    if fused.linear_bias_supported(X2, W, bias):
        out = cuda_bindings.pam_linear(X2, W, bias, offset=offset, approx_bwd=approx_bwd)
        return out.reshape(*lead, out.shape[-1])
    out = matmul(X2, W.T, offset=offset, approx_bwd=approx_bwd)
    out = out.reshape(*lead, out.shape[-1])
    return out if bias is None else out + bias


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def _conv_geometry(X, W, stride, padding, dilation):
    H_in, W_in = X.shape[-2:]
    kH, kW = W.shape[-2:]
    if isinstance(padding, str):
        if padding == "same":
            assert kH % 2 == 1 and kW % 2 == 1
            padding = ((kH - 1) // 2, (kW - 1) // 2)
        elif padding == "valid":
            padding = 0
        else:
            raise ValueError(f"Unknown {padding=}")
    padding, stride = _pair(padding), _pair(stride)
    # the output size formula of the reference ignores dilation (pam_ops.py:140-141)
    H_out = (H_in + 2 * padding[0] - (kH - 1) - 1) // stride[0] + 1
    W_out = (W_in + 2 * padding[1] - (kW - 1) - 1) // stride[1] + 1
    return padding, stride, H_out, W_out


def _patches(X, kernel, padding, stride, dilation, H_out, W_out):
    """[N * locations, C*kH*kW] matrix of the receptive fields, columns ordered (channel, row,
    column) like F.unfold.  Non-overlapping patches (stride = kernel, no padding or dilation: a
    ViT patch embedding) are a reshape and one permuted copy, whose backward is again a permuted
    copy; the general case goes through unfold, whose backward is a scatter-add (fold)."""
    N, C, H, Wd = X.shape
    kH, kW = kernel
    if stride == kernel and padding == (0, 0) and dilation == (1, 1) and H == H_out * kH and Wd == W_out * kW:
        return X.reshape(N, C, H_out, kH, W_out, kW).permute(0, 2, 4, 1, 3, 5).reshape(N * H_out * W_out, C * kH * kW)
    cols = torch.nn.functional.unfold(X, kernel, padding=padding, stride=stride, dilation=dilation)
    return cols.transpose(1, 2).reshape(-1, cols.shape[1])


def conv2d(X, W, bias=None, stride=1, padding=0, dilation=1, *, offset=None, approx_bwd=False, use_kernel=True):
    """Convolution as unfold + PAM linear (pam/pam_ops.py:118-161)."""
    N = X.shape[0]
    C_out, _, kH, kW = W.shape
    padding, stride, H_out, W_out = _conv_geometry(X, W, stride, padding, dilation)
    patches = _patches(X, (kH, kW), padding, stride, _pair(dilation), H_out, W_out)
    Y = linear(patches, W.view(C_out, -1), offset=offset, approx_bwd=approx_bwd)
    Y = Y.view(N, -1, C_out).transpose(1, 2).reshape(N, C_out, H_out, W_out)
    return Y if bias is None else Y + bias.view(1, -1, 1, 1)


def conv2d_group(X, W, bias=None, stride=1, padding=0, dilation=1, groups=1, *,
                 offset=None, approx_bwd=False, use_kernel=True):
    """Grouped convolution as unfold + PAM bmm over the groups (pam/pam_ops.py:164-198)."""
    N, C = X.shape[:2]
    K, _, R, S = W.shape
    G = groups
    padding, stride, H_out, W_out = _conv_geometry(X, W, stride, padding, dilation)
    cols = torch.nn.functional.unfold(X, kernel_size=(R, S), padding=padding, stride=stride, dilation=dilation)
    cols = cols.view(N, G, C // G * R * S, -1).permute(1, 2, 0, 3).reshape(G, C // G * R * S, -1)
    Y = bmm(W.view(G, K // G, C // G * R * S), cols, offset=offset, approx_bwd=approx_bwd)
    Y = Y.view(K, N, H_out, W_out).transpose(0, 1)
    return Y if bias is None else Y + bias.view(1, -1, 1, 1)


class _PamModule:
    """Shared by the three modules: the extra constructor keywords and the ``pam.`` name prefix
    (pam/pam_ops.py:201-285, 381-404)."""

    def _init_pam(self, offset, approx_bwd, use_kernel):
        self.offset, self.approx_bwd, self.use_kernel = offset, approx_bwd, use_kernel

    def _pam_kwargs(self):
        return dict(offset=self.offset, approx_bwd=self.approx_bwd, use_kernel=self.use_kernel)

    def _get_name(self):
        return "pam." + self.__class__.__name__

    def _pam_repr(self, base, with_kernel=False):
        if self.offset is not None:
            base += f", offset={self.offset:0.5f}"
        base += f", approx_bwd={self.approx_bwd}"
        if with_kernel and self.use_kernel is not None:
            base += f", use_kernel={self.use_kernel}"
        return base


class Conv2d(_PamModule, torch.nn.Conv2d):
    def __init__(self, *args, offset=None, approx_bwd=False, use_kernel=True, **kwargs):
        super().__init__(*args, **kwargs)
        self._init_pam(offset, approx_bwd, use_kernel)

    def forward(self, input):
        if self.groups != 1:
            return conv2d_group(input, self.weight, self.bias, self.stride, self.padding, self.dilation,
                                self.groups, **self._pam_kwargs())
        return conv2d(input, self.weight, self.bias, self.stride, self.padding, self.dilation,
                      **self._pam_kwargs())

    def extra_repr(self):
        return self._pam_repr(torch.nn.Conv2d.extra_repr(self))


class Linear(_PamModule, torch.nn.Linear):
    def __init__(self, *args, offset=None, approx_bwd=False, use_kernel=True, **kwargs):
        super().__init__(*args, **kwargs)
        self._init_pam(offset, approx_bwd, use_kernel)

    def forward(self, input):
        return linear(input, self.weight, self.bias, **self._pam_kwargs())

    def extra_repr(self):
        return self._pam_repr(torch.nn.Linear.extra_repr(self))


def mean(input, dim=None, keepdim=False, *, dtype=None, offset=None, approx_bwd=False, use_kernel=True):
    """sum / count with a PAM division (pam/pam_ops.py:288-302)."""
    if dim is None:
        dim = tuple(range(input.dim()))
    if isinstance(dim, int):
        dim = (dim,)
    count = math.prod(input.shape[d] for d in dim)
    return div(torch.sum(input, dim=dim, keepdim=keepdim, dtype=dtype), count,
               offset=offset, approx_bwd=approx_bwd)


_LOG2E = math.log2(math.e)


def softmax(x, dim=None, *, offset=None, approx_bwd=False, use_kernel=True):
    """PAM softmax (pam/pam_ops.py:305-328): x*log2(e) by PAM, exp2 by the piecewise affine
    exponential after subtracting floor(max) of the WHOLE tensor, -inf entries (attention masks)
    forced to probability 0, ordinary sum, PAM division."""
    if fused.softmax_supported(x, dim, approx_bwd):
        return fused.softmax(x, dim, offset=offset, approx_bwd=approx_bwd)
    if x.numel() == 0:              # (the reference fails here: torch.max of an empty tensor)
        return x.clone()
    kw = dict(offset=offset, approx_bwd=approx_bwd)
    masked = x == float("-inf")
    scaled = torch.where(masked, float("-inf"), mul(x, _LOG2E, **kw))
    with torch.no_grad():
        shift = torch.floor(torch.max(scaled))
    e = torch.where(masked, 0, exp2(scaled - shift, **kw))
    return div(e, torch.sum(e, dim=dim, keepdim=True), **kw)


def logsumexp(x, dim, keepdim=False, *, offset=None, approx_bwd=False, use_kernel=True):
    """pam/pam_ops.py:331-342.  As in the reference, the log2 of the row sums runs with the
    default offset and the exact backward whatever this call's settings are."""
    if fused.softmax_supported(x, dim, approx_bwd):
        # the fused route skips the reference's `assert x.isfinite().all()`, which would stall the
        # stream on a device-to-host read; non-finite inputs give NaN there
        return fused.logsumexp(x, dim, keepdim, offset=offset, approx_bwd=approx_bwd)
    kw = dict(offset=offset, approx_bwd=approx_bwd)
    assert x.isfinite().all()
    scaled = mul(x, _LOG2E, **kw)
    with torch.no_grad():
        shift = torch.floor(torch.max(scaled))
    total = torch.sum(exp2(scaled - shift, **kw), dim=dim, keepdim=keepdim)
    return div(shift + log2(total), _LOG2E, **kw)


def log_softmax(x, dim=None, *, offset=None, approx_bwd=False, use_kernel=True):
    return x - logsumexp(x, dim=dim, keepdim=True, offset=offset, approx_bwd=approx_bwd)


def layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-05, *,
               offset=None, approx_bwd=False, use_kernel=True):
    """PAM layer normalisation (pam/pam_ops.py:350-378): PAM mean, PAM square, PAM mean,
    pow(var + eps, 0.5), PAM division, PAM scale, ordinary adds/subtractions."""
    if isinstance(normalized_shape, int):
        normalized_shape = (normalized_shape,)
    normalized_shape = tuple(normalized_shape)
    assert tuple(x.shape[-len(normalized_shape):]) == normalized_shape
    if fused.layer_norm_supported(x, normalized_shape, weight, bias, approx_bwd):
        return fused.layer_norm(x, normalized_shape, weight, bias, eps, offset=offset, approx_bwd=approx_bwd)
    kw = dict(offset=offset, approx_bwd=approx_bwd)
    rows = x.reshape(-1, math.prod(normalized_shape))
    centred = rows - mean(rows, dim=-1, keepdim=True, **kw)
    var = mean(mul(centred, centred, **kw), dim=-1, keepdim=True, **kw)
    out = div(centred, pow(var + eps, 0.5, **kw), **kw).reshape_as(x)
    if weight is not None:
        out = mul(out, weight, **kw)
    return out if bias is None else out + bias


class LayerNorm(_PamModule, torch.nn.LayerNorm):
    def __init__(self, *args, offset=None, approx_bwd=False, use_kernel=True, **kwargs):
        super().__init__(*args, **kwargs)
        self._init_pam(offset, approx_bwd, use_kernel)

    def forward(self, input):
        return layer_norm(input, self.normalized_shape, self.weight, self.bias, self.eps, **self._pam_kwargs())

    def extra_repr(self):
        return self._pam_repr(torch.nn.LayerNorm.extra_repr(self), with_kernel=True)
