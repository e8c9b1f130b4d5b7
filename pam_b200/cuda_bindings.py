"""Kernel bindings and autograd functions — the counterpart of the reference's
``pam/cuda_bindings.py`` with the same public names (``pam pad pam_matmul pam_bmm standard_matmul
pa_exp pa_exp2 pa_log pa_log2 check_row_major cuda_kernels``).

``cuda_kernels`` mirrors the reference's compiled module (pam/cuda_kernels.cu:932-947): fourteen
functions that take CUDA tensors and return a new tensor.  Here they call the sm_100a kernels of
``libpam_b200.so`` through its C ABI.  Differences a caller can observe, all deliberate:

* nothing is compiled at import time (the reference JIT-builds on ``import``);
* kernels run on the tensor's own device and on PyTorch's current stream (the reference uses
  the current device and the legacy default stream);
* broadcast operands (Python numbers, 0-d tensors, row vectors, per-row columns, expanded
  views) are read in place instead of being materialised at full size.
"""
import math

import torch

from . import _lib
from ._lib import COL, FULL, IMM, ROW, SCALAR

# When True, matrix products never split K: every output is summed strictly in k order and the
# result is bit-identical to the reference kernel's.  When False the library may cut K into
# ranges for small outputs (same products, different association of the fp32 sum).
_strict_k_order = False


def set_strict_k_order(flag=True):
    global _strict_k_order
    _strict_k_order = bool(flag)


def strict_k_order():
    return _strict_k_order


def _offset(offset):
    return 1.0 if offset is None else float(offset)   # 1.0 turns the offset off (cuda_bindings.py:31-32)


# ------------------------------------------------------------------------------------------------
# operand description for the elementwise kernels
# ------------------------------------------------------------------------------------------------

def _unexpand(t):
    """Drops broadcast (stride-0) dimensions of an expanded view back to size 1."""
    if t.dim() and any(st == 0 and s > 1 for s, st in zip(t.shape, t.stride())):
        t = t[tuple(slice(0, 1) if st == 0 and s > 1 else slice(None) for s, st in zip(t.shape, t.stride()))]
    return t


class _Desc:
    __slots__ = ("tensor", "kind", "imm", "inner")

    def __init__(self, tensor, kind, imm=0.0, inner=None):
        self.tensor, self.kind, self.imm, self.inner = tensor, kind, imm, inner

    def args(self):
        return (self.tensor.data_ptr() if self.tensor is not None else None, self.kind, self.imm)


def _describe(value, out_shape):
    if isinstance(value, (int, float)):
        return _Desc(None, IMM, float(value))
    t = _unexpand(value.detach())
    if t.dtype != torch.float32:
        t = t.float()
    if t.numel() == 1:
        return _Desc(t.reshape(1), SCALAR)
    nd = len(out_shape)
    shape = (1,) * (nd - t.dim()) + tuple(t.shape)
    if shape == tuple(out_shape):
        return _Desc(t.contiguous(), FULL)
    for j in range(1, nd):
        inner = math.prod(out_shape[j:])
        if all(s == 1 for s in shape[:j]) and shape[j:] == tuple(out_shape[j:]):
            return _Desc(t.contiguous(), ROW, inner=inner)
        if all(s == 1 for s in shape[j:]) and shape[:j] == tuple(out_shape[:j]):
            return _Desc(t.contiguous(), COL, inner=inner)
    return _Desc(t.expand(out_shape).contiguous(), FULL)


def _elementwise(name, operands, offset):
    """out = op(operands...) with NumPy-style broadcasting; operands are tensors or numbers."""
    device = _lib.require_cuda(*operands)
    out_shape = torch.broadcast_shapes(*[o.shape for o in operands if isinstance(o, torch.Tensor)])
    descs = [_describe(o, out_shape) for o in operands]
    inner = None
    for i, d in enumerate(descs):
        if d.inner is None:
            continue
        if inner is None:
            inner = d.inner
        elif d.inner != inner:            # two different row/column splits: expand this one
            descs[i] = _Desc(operands[i].detach().float().expand(out_shape).contiguous(), FULL)
    out = torch.empty(out_shape, dtype=torch.float32, device=device)
    flat = []
    for d in descs:
        flat.extend(d.args())
    with _lib.device_guard(device):
        status = getattr(_lib.lib(), name)(*flat, out.data_ptr(), out.numel(), inner or 0, offset,
                                           _lib.stream_ptr(device))
    _lib.check(status, name)
    return out


def _unary(name, X, *rest, base, offset):
    device = _lib.require_cuda(X, *rest)
    ins = [t.detach().float().contiguous() for t in (X, *rest)]
    for t in ins[1:]:
        if t.shape != ins[0].shape:
            raise ValueError(f"{name}: shapes differ: {tuple(ins[0].shape)} vs {tuple(t.shape)}")
    out = torch.empty_like(ins[0])
    with _lib.device_guard(device):
        status = getattr(_lib.lib(), name)(*[t.data_ptr() for t in ins], out.data_ptr(), out.numel(),
                                           float(base), offset, _lib.stream_ptr(device))
    _lib.check(status, name)
    return out


# ------------------------------------------------------------------------------------------------
# matrix operands
# ------------------------------------------------------------------------------------------------

def check_row_major(tensor, target_dim):
    """(tensor, row_major) as in pam/cuda_bindings.py:106-115: a matrix whose last stride is 1 is
    used as is, one whose second-to-last stride is 1 is used as is and flagged column-major, any
    other layout is copied."""
    if tensor.dim() != target_dim:
        raise ValueError(f"{tensor.dim()=} is not equal to {target_dim=}")
    if tensor.stride()[-1] == 1:
        return tensor, True
    if tensor.stride()[-2] == 1:
        return tensor, False
    return tensor.contiguous(), True


def _matrix(t, dims):
    t, _ = check_row_major(t.detach() if t.dtype == torch.float32 else t.detach().float(), dims)
    if dims == 2:
        return t, (0, t.stride(0), t.stride(1))
    return t, tuple(t.stride())


_workspaces = {}


def _workspace(device, nbytes):
    """Scratch for split-K partial sums, one buffer per (device, stream), grown on demand."""
    key = (device, _lib.stream_ptr(device))
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _matmul(kind, A, B, offset, dims, split_k=None, bias=None):
    device = _lib.require_cuda(A, B)
    A, sa = _matrix(A, dims)
    B, sb = _matrix(B, dims)
    if dims == 3 and A.shape[0] != B.shape[0]:
        raise ValueError(f"batch sizes differ: {A.shape[0]} vs {B.shape[0]}")
    if A.shape[-1] != B.shape[-2]:
        raise ValueError(f"inner dimensions differ: {tuple(A.shape)} x {tuple(B.shape)}")
    batch = A.shape[0] if dims == 3 else 1
    M, K, N = A.shape[-2], A.shape[-1], B.shape[-1]
    out = torch.empty((batch, M, N) if dims == 3 else (M, N), dtype=torch.float32, device=device)
    handle = _lib.lib()
    if split_k is None:
        # (the true-multiply product has one tile shape and its own cost model: it is never split here)
        split_k = 1 if _strict_k_order or kind != _lib.MUL_PAM else handle.pamk_matmul_auto_split(batch, M, N, K)
    ws_ptr, ws_bytes = None, 0
    if split_k > 1:
        ws_bytes = handle.pamk_matmul_workspace_bytes(batch, M, N, split_k)
        ws_ptr = _workspace(device, ws_bytes).data_ptr()
    with _lib.device_guard(device):
        if bias is None:
            status = handle.pamk_matmul(kind, A.data_ptr(), B.data_ptr(), out.data_ptr(), batch, M, N, K,
                                        sa[0], sa[1], sa[2], sb[0], sb[1], sb[2], offset, split_k,
                                        ws_ptr, ws_bytes, _lib.stream_ptr(device))
        else:
            status = handle.pamk_matmul_bias(kind, A.data_ptr(), B.data_ptr(), bias.data_ptr(), out.data_ptr(),
                                             batch, M, N, K, sa[0], sa[1], sa[2], sb[0], sb[1], sb[2], offset,
                                             split_k, ws_ptr, ws_bytes, _lib.stream_ptr(device))
    _lib.check(status, "pamk_matmul")
    return out


def _column_sum(X):
    """Sum over the rows of a 2-D tensor (the bias gradient of a linear layer)."""
    device = _lib.require_cuda(X)
    X = X.detach().float().contiguous()
    rows, cols = X.shape
    out = torch.empty(cols, dtype=torch.float32, device=device)
    handle = _lib.lib()
    ws_bytes = handle.pamk_column_sum_workspace_bytes(rows, cols)
    ws = _workspace(device, ws_bytes) if ws_bytes else None
    with _lib.device_guard(device):
        status = handle.pamk_column_sum(X.data_ptr(), out.data_ptr(), rows, cols,
                                        ws.data_ptr() if ws is not None else None, ws_bytes, _lib.stream_ptr(device))
    _lib.check(status, "pamk_column_sum")
    return out


def _matmul_bwd(L, R, D, delta_l, offset, dims, split_k=None):
    device = _lib.require_cuda(L, R, D)
    L, sl = _matrix(L, dims)
    R, sr = _matrix(R, dims)
    D = D.detach().float()
    sd = (0, D.stride(0), D.stride(1)) if dims == 2 else tuple(D.stride())
    batch = L.shape[0] if dims == 3 else 1
    M, K, N = L.shape[-2], L.shape[-1], R.shape[-1]
    if R.shape[-2] != K or tuple(D.shape[-2:]) != (M, N):
        raise ValueError(f"shape mismatch: {tuple(L.shape)} x {tuple(R.shape)} vs {tuple(D.shape)}")
    out = torch.empty((batch, M, N) if dims == 3 else (M, N), dtype=torch.float32, device=device)
    handle = _lib.lib()
    if split_k is None:
        split_k = 1 if _strict_k_order else handle.pamk_matmul_bwd_auto_split(batch, M, N, K)
    ws_ptr, ws_bytes = None, 0
    if split_k > 1:
        ws_bytes = handle.pamk_matmul_workspace_bytes(batch, M, N, split_k)
        ws_ptr = _workspace(device, ws_bytes).data_ptr()
    with _lib.device_guard(device):
        status = handle.pamk_matmul_bwd(L.data_ptr(), R.data_ptr(), D.data_ptr(), out.data_ptr(),
                                        batch, M, N, K, *sl, *sr, *sd, int(bool(delta_l)), offset,
                                        split_k, ws_ptr, ws_bytes, _lib.stream_ptr(device))
    _lib.check(status, "pamk_matmul_bwd")
    return out


class _CudaKernels:
    """Stand-in for the reference's compiled ``cuda_kernels`` module: same fourteen functions,
    same arguments (pam/cuda_kernels.cu:932-947).  The row-major flags are accepted for
    compatibility; the layout is read from the tensors' strides."""

    @staticmethod
    def pam_fwd(A, B, offset):
        return _elementwise("pamk_pam_fwd", (A, B), offset)

    @staticmethod
    def pam_bwd(A, B, delta_C, offset):
        return _elementwise("pamk_pam_bwd", (A, B, delta_C), offset)

    @staticmethod
    def pad_fwd(A, B, offset):
        return _elementwise("pamk_pad_fwd", (A, B), offset)

    @staticmethod
    def pad_bwd(A, B, delta_C, offset):
        return _elementwise("pamk_pad_bwd", (A, B, delta_C), offset)

    @staticmethod
    def pam_matmul_fwd(A, B, A_row_major=True, B_row_major=True, offset=1.0):
        return _matmul(_lib.MUL_PAM, A, B, offset, 2)

    @staticmethod
    def pam_bmm_fwd(A, B, A_row_major=True, B_row_major=True, offset=1.0):
        return _matmul(_lib.MUL_PAM, A, B, offset, 3)

    @staticmethod
    def pam_matmul_bwd(L, R, M, L_row_major=True, R_row_major=True, delta_L=True, offset=1.0):
        return _matmul_bwd(L, R, M, delta_L, offset, 2)

    @staticmethod
    def pam_bmm_bwd(L, R, M, L_row_major=True, R_row_major=True, delta_L=True, offset=1.0):
        return _matmul_bwd(L, R, M, delta_L, offset, 3)

    @staticmethod
    def standard_matmul(A, B, A_row_major=True, B_row_major=True, offset=1.0):
        return _matmul(_lib.MUL_STANDARD, A, B, 1.0, 2)

    @staticmethod
    def standard_bmm(A, B, A_row_major=True, B_row_major=True, offset=1.0):
        return _matmul(_lib.MUL_STANDARD, A, B, 1.0, 3)

    @staticmethod
    def pa_exp_fwd(X, base, offset):
        return _unary("pamk_pa_exp_fwd", X, base=base, offset=offset)

    @staticmethod
    def pa_exp_bwd(X, dY, base, offset):
        return _unary("pamk_pa_exp_bwd", X, dY, base=base, offset=offset)

    @staticmethod
    def pa_log_fwd(X, base, offset):
        return _unary("pamk_pa_log_fwd", X, base=base, offset=offset)

    @staticmethod
    def pa_log_bwd(X, dY, base, offset):
        return _unary("pamk_pa_log_bwd", X, dY, base=base, offset=offset)


cuda_kernels = _CudaKernels()


# ------------------------------------------------------------------------------------------------
# autograd functions: which kernel runs forward and for each operand's gradient
# (the pairing of pam/cuda_bindings.py:27-57, 66-97, 118-166, 210-239, 250-276)
# ------------------------------------------------------------------------------------------------

def _pair(approx_bwd):
    return (approx_bwd, approx_bwd) if isinstance(approx_bwd, bool) else tuple(approx_bwd)


def _reduce_to(grad, like):
    """Sums a broadcast gradient back to the operand's shape (autograd does this for the
    reference, which expands its operands before the kernel call)."""
    return grad.sum_to_size(like.shape) if tuple(grad.shape) != tuple(like.shape) else grad


def _stash(ctx, *operands):
    """Remembers operands for backward: tensors through save_for_backward, numbers on ctx."""
    ctx.save_for_backward(*[o for o in operands if isinstance(o, torch.Tensor)])
    ctx.numbers = [None if isinstance(o, torch.Tensor) else o for o in operands]


def _unstash(ctx):
    saved = iter(ctx.saved_tensors)
    return [next(saved) if n is None else n for n in ctx.numbers]


class _Mul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, A, B, offset, approx):
        _stash(ctx, A, B)
        ctx.cfg = (offset, approx)
        return cuda_kernels.pam_fwd(A, B, offset)

    @staticmethod
    def backward(ctx, g):
        A, B = _unstash(ctx)
        offset, (approx_a, approx_b) = ctx.cfg
        dA = dB = None
        if ctx.needs_input_grad[0]:
            dA = cuda_kernels.pam_fwd(g, B, offset) if approx_a else cuda_kernels.pam_bwd(A, B, g, offset)
            dA = _reduce_to(dA, A)
        if ctx.needs_input_grad[1]:
            dB = cuda_kernels.pam_fwd(g, A, offset) if approx_b else cuda_kernels.pam_bwd(B, A, g, offset)
            dB = _reduce_to(dB, B)
        return dA, dB, None, None


class _Div(torch.autograd.Function):
    @staticmethod
    def forward(ctx, A, B, offset, approx):
        _stash(ctx, A, B)
        ctx.cfg = (offset, approx)
        return cuda_kernels.pad_fwd(A, B, offset)

    @staticmethod
    def backward(ctx, g):
        A, B = _unstash(ctx)
        offset, (approx_a, approx_b) = ctx.cfg
        dA = dB = None
        if ctx.needs_input_grad[0]:
            recip = cuda_kernels.pad_fwd(1.0, B, offset) if isinstance(B, torch.Tensor) else _host_recip(B, A, offset)
            dA = (cuda_kernels.pam_fwd(recip, g, offset) if approx_a
                  else cuda_kernels.pam_bwd(A, recip, g, 1.0))
            dA = _reduce_to(dA, A)
        if ctx.needs_input_grad[1]:
            if approx_b:
                q2 = cuda_kernels.pad_fwd(cuda_kernels.pad_fwd(A, B, offset), B, offset)
                dB = -cuda_kernels.pam_fwd(q2, g, offset)
            else:
                dB = cuda_kernels.pad_bwd(A, B, g, offset)
            dB = _reduce_to(dB, B)
        return dA, dB, None, None


def _host_recip(b, like, offset):
    """pad(1, b) for a Python-number divisor, evaluated by the kernel on a one-element tensor."""
    one = torch.ones(1, dtype=torch.float32, device=like.device)
    return cuda_kernels.pad_fwd(one, b, offset)


class _Exp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, base, offset, approx):
        ctx.save_for_backward(X)
        ctx.cfg = (base, offset, approx)
        return cuda_kernels.pa_exp_fwd(X, base, offset)

    @staticmethod
    def backward(ctx, g):
        (X,) = ctx.saved_tensors
        base, offset, approx = ctx.cfg
        if not approx:
            return cuda_kernels.pa_exp_bwd(X, g.contiguous(), base, offset), None, None, None
        Y = cuda_kernels.pa_exp_fwd(X, base, offset)
        if base != math.e:
            Y = cuda_kernels.pam_fwd(Y, math.log(base), offset)
        return cuda_kernels.pam_fwd(Y, g, offset), None, None, None


class _Log(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, base, offset, approx):
        ctx.save_for_backward(X)
        ctx.cfg = (base, offset, approx)
        return cuda_kernels.pa_log_fwd(X, base, offset)

    @staticmethod
    def backward(ctx, g):
        (X,) = ctx.saved_tensors
        base, offset, approx = ctx.cfg
        if not approx:
            return cuda_kernels.pa_log_bwd(X, g.contiguous(), base, offset), None, None, None
        dX = cuda_kernels.pad_fwd(g, X, offset)
        if base != math.e:
            dX = cuda_kernels.pad_fwd(dX, math.log(base), offset)
        return dX, None, None, None


class _MatMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, A, B, offset, approx, bmm):
        ctx.save_for_backward(A, B)
        ctx.cfg = (offset, approx, bmm)
        return _matmul(_lib.MUL_PAM, A, B, offset, 3 if bmm else 2)

    @staticmethod
    def backward(ctx, g):
        A, B = ctx.saved_tensors
        offset, (approx_a, approx_b), bmm = ctx.cfg
        dims = 3 if bmm else 2
        dA = dB = None
        if ctx.needs_input_grad[0]:
            dA = (_matmul(_lib.MUL_PAM, g, B.mT, offset, dims) if approx_a
                  else _matmul_bwd(g, B.mT, A, True, offset, dims))
        if ctx.needs_input_grad[1]:
            dB = (_matmul(_lib.MUL_PAM, A.mT, g, offset, dims) if approx_b
                  else _matmul_bwd(A.mT, g, B, False, offset, dims))
        return dA, dB, None, None, None


class _Linear(torch.autograd.Function):
    """X @ W.T + bias in one launch (the bias is added in the product's epilogue with the same
    ordinary add the reference issues separately, pam/pam_ops.py:107-115); the gradients are those
    of _MatMul for X and W.T, and the column sum of the incoming gradient for the bias."""

    @staticmethod
    def forward(ctx, X, W, bias, offset, approx):
        ctx.save_for_backward(X, W)
        ctx.cfg = (offset, approx)
        return _matmul(_lib.MUL_PAM, X, W.T, offset, 2, bias=bias)

    @staticmethod
    def backward(ctx, g):
        X, W = ctx.saved_tensors
        offset, (approx_a, approx_b) = ctx.cfg
        dX = dW = db = None
        if ctx.needs_input_grad[0]:
            dX = _matmul(_lib.MUL_PAM, g, W, offset, 2) if approx_a else _matmul_bwd(g, W, X, True, offset, 2)
        if ctx.needs_input_grad[1]:
            dWt = (_matmul(_lib.MUL_PAM, X.mT, g, offset, 2) if approx_b
                   else _matmul_bwd(X.mT, g, W.T, False, offset, 2))
            dW = dWt.T
        if ctx.needs_input_grad[2]:
            db = _column_sum(g)
        return dX, dW, db, None, None


class _StandardMatMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, A, B, bmm):
        ctx.save_for_backward(A, B)
        ctx.bmm = bmm
        return _matmul(_lib.MUL_STANDARD, A, B, 1.0, 3 if bmm else 2)

    @staticmethod
    def backward(ctx, g):
        A, B = ctx.saved_tensors
        dims = 3 if ctx.bmm else 2
        dA = _matmul(_lib.MUL_STANDARD, g, B.mT, 1.0, dims) if ctx.needs_input_grad[0] else None
        dB = _matmul(_lib.MUL_STANDARD, A.mT, g, 1.0, dims) if ctx.needs_input_grad[1] else None
        return dA, dB, None


# ---- public functions (names and keyword arguments of pam/cuda_bindings.py) ----------------------

def _as_operand(v, device):
    """Tensors pass through; Python numbers stay numbers (passed by value to the kernel)."""
    if isinstance(v, torch.Tensor):
        return v
    if isinstance(v, (int, float)):
        return float(v)
    raise TypeError(f"unsupported operand type {type(v)}")


def pam(A, B, *, offset=None, approx_bwd=False):
    _lib.require_cuda(A, B)
    return _Mul.apply(_as_operand(A, None), _as_operand(B, None), _offset(offset), _pair(approx_bwd))


def pad(A, B, *, offset=None, approx_bwd=False):
    _lib.require_cuda(A, B)
    if not isinstance(A, torch.Tensor):          # number / tensor: give the kernel a tensor dividend
        A = torch.full((1,), float(A), dtype=torch.float32, device=B.device)
    return _Div.apply(A, _as_operand(B, None), _offset(offset), _pair(approx_bwd))


def pam_matmul(A, B, *, offset=None, approx_bwd=False):
    return _MatMul.apply(A, B, _offset(offset), _pair(approx_bwd), False)


def pam_linear(X, W, bias, *, offset=None, approx_bwd=False):
    """[rows, in] x [out, in] + [out] (no counterpart in the reference's bindings: its `linear` is
    pam_matmul followed by a torch add)."""
    return _Linear.apply(X, W, bias, _offset(offset), _pair(approx_bwd))


def pam_bmm(A, B, *, offset=None, approx_bwd=False):
    return _MatMul.apply(A, B, _offset(offset), _pair(approx_bwd), True)


def standard_matmul(A, B, *, offset=None, approx_bwd=None, BMM=False):
    return _StandardMatMul.apply(A, B, BMM)


def pa_exp(X, *, base=math.e, offset=None, approx_bwd=False):
    return _Exp.apply(X, base, _offset(offset), approx_bwd)


def pa_exp2(X, *, offset=None, approx_bwd=False):
    return _Exp.apply(X, 2.0, _offset(offset), approx_bwd)


def pa_log(X, *, base=math.e, offset=None, approx_bwd=False):
    return _Log.apply(X, base, _offset(offset), approx_bwd)


def pa_log2(X, *, offset=None, approx_bwd=False):
    return _Log.apply(X, 2.0, _offset(offset), approx_bwd)
