"""Test-only stand-in for libpam_b200.so that evaluates the C ABI on HOST memory with the CPU
oracle.  It lets the `-m "not gpu"` tests exercise the Python host layer (operand description,
broadcasting, autograd pairing, shapes, strides) on a machine without a GPU.  It is installed by
the `cpu_backend` fixture through monkeypatching and is never importable from the package."""
import contextlib
import ctypes

import numpy as np
import torch

from oracle import pam_oracle

FULL, SCALAR, ROW, COL, IMM = range(5)


def _view(ptr, count):
    return np.ctypeslib.as_array((ctypes.c_float * count).from_address(ptr))


class FakeLib:
    def __init__(self):
        self.o = pam_oracle.kernels().lib
        self.calls = []

    def _operand(self, ptr, kind, imm, n, inner):
        if kind == IMM:
            return np.full(n, np.float32(imm), dtype=np.float32)
        if kind == SCALAR:
            return np.full(n, _view(ptr, 1)[0], dtype=np.float32)
        if kind == FULL:
            return np.array(_view(ptr, n))
        if kind == ROW:
            return np.tile(_view(ptr, inner), n // inner)
        if kind == COL:
            return np.repeat(_view(ptr, n // inner), inner)
        raise ValueError(kind)

    def _ew(self, fn, nin, args):
        ops, rest = args[:3 * nin], args[3 * nin:]
        out, n, inner, offset, _stream = rest
        self.calls.append((fn, [ops[3 * i + 1] for i in range(nin)], n, inner))
        if n == 0:
            return 0
        arrs = [self._operand(ops[3 * i], ops[3 * i + 1], ops[3 * i + 2], n, inner) for i in range(nin)]
        res = np.empty(n, dtype=np.float32)
        getattr(self.o, fn)(*[a.ctypes.data for a in arrs], res.ctypes.data, n, pam_oracle.offset_to_int(offset))
        _view(out, n)[:] = res
        return 0

    def pamk_pam_fwd(self, *a): return self._ew("orc_pam", 2, a)
    def pamk_pad_fwd(self, *a): return self._ew("orc_pad", 2, a)
    def pamk_pam_bwd(self, *a): return self._ew("orc_pam_bwd", 3, a)
    def pamk_pad_bwd(self, *a): return self._ew("orc_pad_bwd", 3, a)

    def _unary(self, fn, ptrs, n, base, offset):
        self.calls.append((fn, n))
        if n:
            getattr(self.o, fn)(*ptrs, n, base, pam_oracle.offset_to_int(offset))
        return 0

    def pamk_pa_exp_fwd(self, x, y, n, base, offset, s): return self._unary("orc_pa_exp", (x, y), n, base, offset)
    def pamk_pa_exp_bwd(self, x, dy, dx, n, base, offset, s): return self._unary("orc_pa_exp_bwd", (x, dy, dx), n, base, offset)
    def pamk_pa_log_fwd(self, x, y, n, base, offset, s): return self._unary("orc_pa_log", (x, y), n, base, offset)
    def pamk_pa_log_bwd(self, x, dy, dx, n, base, offset, s): return self._unary("orc_pa_log_bwd", (x, dy, dx), n, base, offset)

    def pamk_matmul_auto_split(self, batch, M, N, K): return 1
    def pamk_matmul_bwd_auto_split(self, batch, M, N, K): return 1
    def pamk_matmul_workspace_bytes(self, batch, M, N, split): return 0

    def pamk_matmul(self, kind, A, B, C, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, offset, split, ws, wsb, s):
        self.calls.append(("matmul", kind, (batch, M, N, K), (sAb, sAm, sAk), (sBb, sBk, sBn)))
        for sm, sk, rows in ((sAm, sAk, M), (sBn, sBk, N)):
            if not (sk == 1 or K == 1 or sm == 1 or rows == 1):
                return -3
        self.o.orc_matmul(A, B, C, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, kind, pam_oracle.offset_to_int(offset))
        return 0

    def pamk_matmul_bias(self, kind, A, B, bias, C, batch, M, N, K, *rest):
        status = self.pamk_matmul(kind, A, B, C, batch, M, N, K, *rest)
        if status == 0 and bias and batch * M * N:
            out = _view(C, batch * M * N).reshape(batch * M, N)
            out += _view(bias, N)                       # one fp32 add per element, after the sum
        return status

    def pamk_column_sum_workspace_bytes(self, rows, cols): return 0

    def pamk_column_sum(self, X, out, rows, cols, ws, wsb, s):
        # torch's CPU sum, so that host-layer results keep the reference's own reduction
        _view(out, cols)[:] = torch.from_numpy(_view(X, rows * cols).reshape(rows, cols)).sum(0).numpy() if rows else 0.0
        return 0

    def pamk_matmul_bwd(self, L, R, D, C, batch, M, N, K, *rest):
        strides, (delta_l, offset, _split, _ws, _wsb, _s) = rest[:9], rest[9:]
        self.calls.append(("matmul_bwd", (batch, M, N, K), strides, delta_l))
        self.o.orc_matmul_bwd(L, R, D, C, batch, M, N, K, *strides, delta_l, pam_oracle.offset_to_int(offset))
        return 0

    def pamk_status_string(self, status): return b"fake backend error"
    def pamk_last_cuda_error(self): return 0


def install(monkeypatch):
    from pam_b200 import _lib, pam_ops
    fake = FakeLib()

    def require(*tensors):
        devs = {t.device for t in tensors if isinstance(t, torch.Tensor)}
        assert len(devs) == 1, devs
        return devs.pop()

    monkeypatch.setattr(_lib, "lib", lambda: fake)
    monkeypatch.setattr(_lib, "require_cuda", require)
    monkeypatch.setattr(_lib, "stream_ptr", lambda device: 0)
    monkeypatch.setattr(_lib, "device_guard", lambda device: contextlib.nullcontext())
    monkeypatch.setattr(pam_ops, "_scalar_device", lambda: torch.device("cpu"))
    return fake
