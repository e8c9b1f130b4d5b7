"""TEST INFRASTRUCTURE — CPU oracle for the PAM hot path (never imported by the shipped package).

Layers, bottom up:

* ``CpuKernels``  — the 14 entry points the reference exposes at its native boundary
  (epfml/pam pam/cuda_kernels.cu:932-947), evaluated on CPU tensors by ``libpam_oracle.so``
  (the C restatement, kind ``"port"``) or by ``_ref/libpam_ref.so`` (the reference's own scalar
  functions compiled for the host, kind ``"reference"``).
* autograd primitives ``mul div exp exp2 log log2 matmul bmm`` — the forward/backward pairing of
  pam/cuda_bindings.py:27-283 (approximate vs exact backward per operand).
* composites ``pow mean softmax logsumexp log_softmax layer_norm linear`` — pam/pam_ops.py:70-378,
  and ``adam_step`` — submodules/fairseq/fairseq/optim/adam.py:226-252.

Parity status: pinned for pam/matmul by the reference's known-answer vectors
(pam/test_pam.py:13-29,36-43,96-97,129-130); every primitive is additionally compared bit-for-bit
with the reference's host-compiled scalar functions, and the composites with the reference's own
Python (pam_ops.py / cuda_bindings.py run over those functions) through the committed fixtures in
tests/golden/.  The reference has no test of its own for pad, exp/log, pow, softmax, layer_norm
or Adam.
"""
import ctypes
import math
import pathlib
import struct

import torch

_HERE = pathlib.Path(__file__).resolve().parent
_i64, _int, _flt = ctypes.c_int64, ctypes.c_int, ctypes.c_float
_ptr = ctypes.c_void_p


def offset_to_int(offset):
    """float offset -> integer added to the bit pattern (pam/cuda_kernels.cu:168); None means 1.0."""
    if offset is None:
        offset = 1.0
    return struct.unpack("<i", struct.pack("<f", float(offset)))[0] - 0x3F800000


def _load(path):
    lib = ctypes.CDLL(str(path))
    ew2 = [_ptr, _ptr, _ptr, _i64, _int]
    ew3 = [_ptr, _ptr, _ptr, _ptr, _i64, _int]
    lib.orc_pam.argtypes = ew2
    lib.orc_pad.argtypes = ew2
    lib.orc_pam_bwd.argtypes = ew3
    lib.orc_pad_bwd.argtypes = ew3
    lib.orc_pa_exp.argtypes = [_ptr, _ptr, _i64, _flt, _int]
    lib.orc_pa_log.argtypes = [_ptr, _ptr, _i64, _flt, _int]
    lib.orc_pa_exp_bwd.argtypes = [_ptr, _ptr, _ptr, _i64, _flt, _int]
    lib.orc_pa_log_bwd.argtypes = [_ptr, _ptr, _ptr, _i64, _flt, _int]
    lib.orc_matmul.argtypes = [_ptr] * 3 + [_i64] * 10 + [_int, _int]
    lib.orc_matmul_bwd.argtypes = [_ptr] * 4 + [_i64] * 13 + [_int, _int]
    lib.orc_set_threads.argtypes = [_int]
    lib.orc_max_threads.restype = _int
    for name in ("orc_pam", "orc_pad", "orc_pam_bwd", "orc_pad_bwd", "orc_pa_exp", "orc_pa_log",
                 "orc_pa_exp_bwd", "orc_pa_log_bwd", "orc_matmul", "orc_matmul_bwd", "orc_set_threads"):
        getattr(lib, name).restype = None
    return lib


def library_path(kind="port"):
    return _HERE / ("libpam_oracle.so" if kind == "port" else "_ref/libpam_ref.so")


def _flat(t):
    t = t.detach()
    assert t.device.type == "cpu"
    return t.to(torch.float32).contiguous().view(-1)


class CpuKernels:
    """CPU stand-in for the reference's ``cuda_kernels`` module (same names, same arguments)."""

    def __init__(self, kind="port"):
        path = library_path(kind)
        if not path.exists():
            raise FileNotFoundError(f"{path} missing: run `python oracle/build.py`")
        self.kind = kind
        self.lib = _load(path)

    def set_threads(self, n):
        self.lib.orc_set_threads(int(n))

    def max_threads(self):
        return self.lib.orc_max_threads()

    # -- elementwise -----------------------------------------------------------------------
    def _ew(self, fn, ins, like, *scalars):
        flats = [_flat(t) for t in ins]
        n = flats[0].numel()
        assert all(f.numel() == n for f in flats)
        out = torch.empty(n, dtype=torch.float32)
        fn(*[f.data_ptr() for f in flats], out.data_ptr(), n, *scalars)
        return out.view(like.shape)

    def pam_fwd(self, A, B, offset):
        return self._ew(self.lib.orc_pam, (A, B), A, offset_to_int(offset))

    def pam_bwd(self, A, B, dC, offset):
        return self._ew(self.lib.orc_pam_bwd, (A, B, dC), A, offset_to_int(offset))

    def pad_fwd(self, A, B, offset):
        return self._ew(self.lib.orc_pad, (A, B), A, offset_to_int(offset))

    def pad_bwd(self, A, B, dC, offset):
        return self._ew(self.lib.orc_pad_bwd, (A, B, dC), A, offset_to_int(offset))

    def pa_exp_fwd(self, X, base, offset):
        return self._ew(self.lib.orc_pa_exp, (X,), X, float(base), offset_to_int(offset))

    def pa_exp_bwd(self, X, dY, base, offset):
        return self._ew(self.lib.orc_pa_exp_bwd, (X, dY), X, float(base), offset_to_int(offset))

    def pa_log_fwd(self, X, base, offset):
        return self._ew(self.lib.orc_pa_log, (X,), X, float(base), offset_to_int(offset))

    def pa_log_bwd(self, X, dY, base, offset):
        return self._ew(self.lib.orc_pa_log_bwd, (X, dY), X, float(base), offset_to_int(offset))

    # -- matrix products (layout flags of the reference are implied by the strides) ---------
    @staticmethod
    def _as3(t):
        t = t.detach().to(torch.float32)
        return t if t.dim() == 3 else t.unsqueeze(0)

    def _mm(self, A, B, mode, offset):
        squeeze = A.dim() == 2
        A3, B3 = self._as3(A), self._as3(B)
        bt, M, K = A3.shape
        assert B3.shape[0] == bt and B3.shape[1] == K
        N = B3.shape[2]
        C = torch.empty(bt, M, N, dtype=torch.float32)
        self.lib.orc_matmul(A3.data_ptr(), B3.data_ptr(), C.data_ptr(), bt, M, N, K,
                            *A3.stride(), *B3.stride(), mode, offset_to_int(offset))
        return C[0] if squeeze else C

    def pam_matmul_fwd(self, A, B, A_rm=True, B_rm=True, offset=1.0):
        return self._mm(A, B, 0, offset)

    pam_bmm_fwd = pam_matmul_fwd

    def standard_matmul(self, A, B, A_rm=True, B_rm=True, offset=1.0):
        return self._mm(A, B, 1, offset)

    standard_bmm = standard_matmul

    def pam_matmul_bwd(self, L, R, D, L_rm=True, R_rm=True, delta_L=True, offset=1.0):
        squeeze = L.dim() == 2
        L3, R3, D3 = self._as3(L), self._as3(R), self._as3(D)
        bt, M, K = L3.shape
        N = R3.shape[2]
        assert R3.shape[:2] == (bt, K) and D3.shape == (bt, M, N)
        C = torch.empty(bt, M, N, dtype=torch.float32)
        self.lib.orc_matmul_bwd(L3.data_ptr(), R3.data_ptr(), D3.data_ptr(), C.data_ptr(), bt, M, N, K,
                                *L3.stride(), *R3.stride(), *D3.stride(), int(bool(delta_L)),
                                offset_to_int(offset))
        return C[0] if squeeze else C

    pam_bmm_bwd = pam_matmul_bwd


_default = None


def kernels(kind="port"):
    global _default
    if kind != "port":
        return CpuKernels(kind)
    if _default is None:
        _default = CpuKernels("port")
    return _default


# ------------------------------------------------------------------------------------------------
# Autograd primitives: which kernel runs in forward and in each operand's backward.
# ------------------------------------------------------------------------------------------------

def _pair(approx_bwd):
    return (approx_bwd, approx_bwd) if isinstance(approx_bwd, bool) else tuple(approx_bwd)


def _tensors(*values):
    """python numbers -> fp32 0-d tensors (pam/utils.py:3-17)."""
    return [torch.tensor(v, dtype=torch.float32) if isinstance(v, (int, float)) else v for v in values]


def _demote(out, ins):
    return out.item() if all(isinstance(v, (int, float)) for v in ins) else out


class _Mul(torch.autograd.Function):
    # pam/cuda_bindings.py:27-57
    @staticmethod
    def forward(ctx, A, B, offset, approx, K):
        ctx.save_for_backward(A, B)
        ctx.cfg = (offset, approx, K)
        return K.pam_fwd(A, B, offset)

    @staticmethod
    def backward(ctx, g):
        A, B = ctx.saved_tensors
        offset, (ax, bx), K = ctx.cfg
        g = g.contiguous()
        dA = K.pam_fwd(g, B, offset) if ax else K.pam_bwd(A, B, g, offset)
        dB = K.pam_fwd(g, A, offset) if bx else K.pam_bwd(B, A, g, offset)
        return dA, dB, None, None, None


class _Div(torch.autograd.Function):
    # pam/cuda_bindings.py:66-97
    @staticmethod
    def forward(ctx, A, B, offset, approx, K):
        ctx.save_for_backward(A, B)
        ctx.cfg = (offset, approx, K)
        return K.pad_fwd(A, B, offset)

    @staticmethod
    def backward(ctx, g):
        A, B = ctx.saved_tensors
        offset, (ax, bx), K = ctx.cfg
        g = g.contiguous()
        recip = K.pad_fwd(torch.ones_like(B), B, offset)
        dA = K.pam_fwd(recip, g, offset) if ax else K.pam_bwd(A, recip, g, 1.0)
        if bx:
            dB = -K.pam_fwd(K.pad_fwd(K.pad_fwd(A, B, offset), B, offset), g, offset)
        else:
            dB = K.pad_bwd(A, B, g, offset)
        return dA, dB, None, None, None


class _Exp(torch.autograd.Function):
    # pam/cuda_bindings.py:210-239
    @staticmethod
    def forward(ctx, X, base, offset, approx, K):
        ctx.save_for_backward(X)
        ctx.cfg = (base, offset, approx, K)
        return K.pa_exp_fwd(X, base, offset)

    @staticmethod
    def backward(ctx, g):
        (X,) = ctx.saved_tensors
        base, offset, approx, K = ctx.cfg
        if not approx:
            return K.pa_exp_bwd(X, g, base, offset), None, None, None, None
        Y = K.pa_exp_fwd(X, base, offset)
        if base != math.e:
            Y = K.pam_fwd(Y, torch.full_like(X, math.log(base)), offset)
        return K.pam_fwd(Y, g, offset), None, None, None, None


class _Log(torch.autograd.Function):
    # pam/cuda_bindings.py:250-276
    @staticmethod
    def forward(ctx, X, base, offset, approx, K):
        ctx.save_for_backward(X)
        ctx.cfg = (base, offset, approx, K)
        return K.pa_log_fwd(X, base, offset)

    @staticmethod
    def backward(ctx, g):
        (X,) = ctx.saved_tensors
        base, offset, approx, K = ctx.cfg
        if not approx:
            return K.pa_log_bwd(X, g, base, offset), None, None, None, None
        dX = K.pad_fwd(g, X, offset)
        if base != math.e:
            dX = K.pad_fwd(dX, torch.full_like(X, math.log(base)), offset)
        return dX, None, None, None, None


class _MatMul(torch.autograd.Function):
    # pam/cuda_bindings.py:118-166 ; mode "pam" or "standard" (:176-201)
    @staticmethod
    def forward(ctx, A, B, offset, approx, mode, K):
        ctx.save_for_backward(A, B)
        ctx.cfg = (offset, approx, mode, K)
        return K.pam_matmul_fwd(A, B, True, True, offset) if mode == "pam" else K.standard_matmul(A, B)

    @staticmethod
    def backward(ctx, g):
        A, B = ctx.saved_tensors
        offset, (ax, bx), mode, K = ctx.cfg
        if mode != "pam":
            return K.standard_matmul(g, B.mT), K.standard_matmul(A.mT, g), None, None, None, None
        dA = (K.pam_matmul_fwd(g, B.mT, True, True, offset) if ax
              else K.pam_matmul_bwd(g, B.mT, A, True, True, True, offset))
        dB = (K.pam_matmul_fwd(A.mT, g, True, True, offset) if bx
              else K.pam_matmul_bwd(A.mT, g, B, True, True, False, offset))
        return dA, dB, None, None, None, None


def _off(offset):
    return 1.0 if offset is None else offset


def mul(A, B, *, offset=None, approx_bwd=False, K=None):
    tA, tB = torch.broadcast_tensors(*_tensors(A, B))
    return _demote(_Mul.apply(tA, tB, _off(offset), _pair(approx_bwd), K or kernels()), (A, B))


def div(A, B, *, offset=None, approx_bwd=False, K=None):
    tA, tB = torch.broadcast_tensors(*_tensors(A, B))
    return _demote(_Div.apply(tA, tB, _off(offset), _pair(approx_bwd), K or kernels()), (A, B))


def exp(A, base=math.e, *, offset=None, approx_bwd=False, K=None):
    (tA,) = _tensors(A)
    return _demote(_Exp.apply(tA, base, _off(offset), approx_bwd, K or kernels()), (A,))


def exp2(A, **kw):
    return exp(A, 2.0, **kw)


def log(A, base=math.e, *, offset=None, approx_bwd=False, K=None):
    (tA,) = _tensors(A)
    return _demote(_Log.apply(tA, base, _off(offset), approx_bwd, K or kernels()), (A,))


def log2(A, **kw):
    return log(A, 2.0, **kw)


def matmul(A, B, *, offset=None, approx_bwd=False, K=None):
    return _MatMul.apply(A, B, _off(offset), _pair(approx_bwd), "pam", K or kernels())


bmm = matmul


def standard_matmul(A, B, *, K=None):
    return _MatMul.apply(A, B, 1.0, (True, True), "standard", K or kernels())


# ------------------------------------------------------------------------------------------------
# Composites (pam/pam_ops.py)
# ------------------------------------------------------------------------------------------------

def pow(A, B, **kw):
    # pam/pam_ops.py:70-79
    tA, tB = _tensors(A, B)
    out = torch.where(tA == 0, 0, exp2(mul(log2(tA, **kw), tB, **kw), **kw))
    return _demote(out, (A, B))


def linear(X, W, bias=None, **kw):
    # pam/pam_ops.py:107-115
    out = matmul(X.reshape(-1, X.shape[-1]), W.T, **kw).reshape(*X.shape[:-1], W.shape[0])
    return out if bias is None else out + bias


def mean(x, dim=None, keepdim=False, **kw):
    # pam/pam_ops.py:288-302
    dims = tuple(range(x.dim())) if dim is None else ((dim,) if isinstance(dim, int) else tuple(dim))
    count = math.prod(x.shape[d] for d in dims)
    return div(torch.sum(x, dim=dims, keepdim=keepdim), count, **kw)


_LOG2E = math.log2(math.e)


def softmax(x, dim=None, **kw):
    # pam/pam_ops.py:305-328 — note the shift is floor(max) over the WHOLE tensor
    masked = x == float("-inf")
    scaled = torch.where(masked, float("-inf"), mul(x, _LOG2E, **kw))
    with torch.no_grad():
        shift = torch.floor(torch.max(scaled))
    e = torch.where(masked, 0, exp2(scaled - shift, **kw))
    return div(e, torch.sum(e, dim=dim, keepdim=True), **kw)


def logsumexp(x, dim, keepdim=False, **kw):
    # pam/pam_ops.py:331-342
    assert x.isfinite().all()
    scaled = mul(x, _LOG2E, **kw)
    with torch.no_grad():
        shift = torch.floor(torch.max(scaled))
    total = torch.sum(exp2(scaled - shift, **kw), dim=dim, keepdim=keepdim)
    # the reference calls log2 here WITHOUT forwarding offset/approx_bwd (pam_ops.py:341):
    # this one primitive always runs with offset None and the exact backward
    return div(shift + log2(total, K=kw.get("K")), _LOG2E, **kw)


def log_softmax(x, dim=None, **kw):
    # pam/pam_ops.py:345-347
    return x - logsumexp(x, dim=dim, keepdim=True, **kw)


def layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5, **kw):
    # pam/pam_ops.py:350-378
    if isinstance(normalized_shape, int):
        normalized_shape = (normalized_shape,)
    width = math.prod(normalized_shape)
    rows = x.reshape(-1, width)
    centred = rows - mean(rows, dim=-1, keepdim=True, **kw)
    var = mean(mul(centred, centred, **kw), dim=-1, keepdim=True, **kw)
    out = div(centred, pow(var + eps, 0.5, **kw), **kw).reshape_as(x)
    if weight is not None:
        out = mul(out, weight, **kw)
    return out if bias is None else out + bias


def adam_step(p, grad, exp_avg, exp_avg_sq, *, step, lr, betas, eps, weight_decay, **kw):
    """One PAM Adam update of one tensor (submodules/fairseq/fairseq/optim/adam.py:226-252).
    ``step`` is the step count AFTER the increment.  Returns new (p, exp_avg, exp_avg_sq)."""
    b1, b2 = betas
    with torch.no_grad():
        m = mul(exp_avg, b1, **kw) + mul(grad, 1 - b1, **kw)
        v = mul(exp_avg_sq, b2, **kw)
        v = v + mul(mul(grad, grad, **kw), 1 - b2, **kw)
        denom = pow(v, 0.5, **kw) + eps
        step_size = lr * math.sqrt(1 - b2 ** step) / (1 - b1 ** step)
        p = p.clone()
        if weight_decay != 0:
            p -= mul(p, weight_decay * lr, **kw)
        p -= mul(div(m, denom, **kw), step_size, **kw)
    return p, m, v
