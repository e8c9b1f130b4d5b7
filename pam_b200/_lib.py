"""ctypes binding of ``libpam_b200.so`` (the C ABI declared in ``include/pam_b200.h``).

There is no fallback: if the library has not been built, or a call returns an error status, an
exception is raised.  PyTorch only supplies device memory and the stream; every operation below
runs in the library's own sm_100a kernels.
"""
import ctypes
import os
import pathlib

import torch

_PKG = pathlib.Path(__file__).resolve().parent
# PAM_B200_LIBRARY points at another build of the same library (A/B comparisons of kernel variants).
LIB_PATH = pathlib.Path(os.environ.get("PAM_B200_LIBRARY") or _PKG / "libpam_b200.so")

FULL, SCALAR, ROW, COL, IMM = 0, 1, 2, 3, 4
MUL_PAM, MUL_STANDARD = 0, 1

_p, _i, _i64, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t
_operand = [_p, _i, _f]

_SIGNATURES = {
    "pamk_status_string": (ctypes.c_char_p, [_i]),
    "pamk_last_cuda_error": (_i, []),
    "pamk_abi_version": (_i, []),
    "pamk_launch_count": (ctypes.c_longlong, []),
    "pamk_pam_fwd": (_i, _operand * 2 + [_p, _i64, _i64, _f, _p]),
    "pamk_pad_fwd": (_i, _operand * 2 + [_p, _i64, _i64, _f, _p]),
    "pamk_pam_bwd": (_i, _operand * 3 + [_p, _i64, _i64, _f, _p]),
    "pamk_pad_bwd": (_i, _operand * 3 + [_p, _i64, _i64, _f, _p]),
    "pamk_pa_exp_fwd": (_i, [_p, _p, _i64, _f, _f, _p]),
    "pamk_pa_exp_bwd": (_i, [_p, _p, _p, _i64, _f, _f, _p]),
    "pamk_pa_log_fwd": (_i, [_p, _p, _i64, _f, _f, _p]),
    "pamk_pa_log_bwd": (_i, [_p, _p, _p, _i64, _f, _f, _p]),
    "pamk_matmul": (_i, [_i, _p, _p, _p] + [_i64] * 10 + [_f, _i, _p, _sz, _p]),
    "pamk_matmul_bias": (_i, [_i, _p, _p, _p, _p] + [_i64] * 10 + [_f, _i, _p, _sz, _p]),
    "pamk_column_sum_workspace_bytes": (_sz, [_i64, _i64]),
    "pamk_column_sum": (_i, [_p, _p, _i64, _i64, _p, _sz, _p]),
    "pamk_matmul_workspace_bytes": (_sz, [_i64, _i64, _i64, _i]),
    "pamk_matmul_auto_split": (_i, [_i64] * 4),
    "pamk_test_set_tile_policy": (_i, [_i]),
    "pamk_test_planned_tile": (_i, [_i64] * 4),
    "pamk_matmul_static_scratch_bytes": (_sz, []),
    "pamk_matmul_static_scratch": (_i, [_p, _p, _p] + [_i64] * 10 + [_f, _i, _p]),
    "pamk_matmul_bwd": (_i, [_p] * 4 + [_i64] * 13 + [_i, _f, _i, _p, ctypes.c_size_t, _p]),
    "pamk_matmul_bwd_auto_split": (_i, [_i64] * 4),
    "pamk_layer_norm_max_width": (_i, []),
    "pamk_layer_norm_fwd": (_i, [_p, _p, _p, _p, _i64, _i64, _f, _f, _p]),
    "pamk_layer_norm_stats_per_row": (_i, []),
    "pamk_layer_norm_fwd_save": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _f, _f, _p]),
    "pamk_layer_norm_bwd_saved": (_i, [_p] * 7 + [_i64, _i64, _f, _p, _sz, _p]),
    "pamk_layer_norm_bwd_workspace_bytes": (_sz, [_i64, _i64]),
    "pamk_layer_norm_bwd": (_i, [_p] * 6 + [_i64, _i64, _f, _f, _i, _p, _sz, _p]),
    "pamk_softmax_max_len": (_i, []),
    "pamk_softmax_workspace_bytes": (_sz, [_i64, _i64]),
    "pamk_softmax_fwd": (_i, [_p, _p, _i64, _i64, _f, _p, _sz, _p]),
    "pamk_softmax_bwd": (_i, [_p, _p, _p, _i64, _i64, _f, _i, _p, _sz, _p]),
    "pamk_softmax_fwd_save": (_i, [_p, _p, _p, _i64, _i64, _f, _p, _sz, _p]),
    "pamk_softmax_bwd_saved": (_i, [_p, _p, _p, _i64, _i64, _f, _i, _f, _p]),
    "pamk_softmax_bwd_scaled": (_i, [_p, _p, _p, _i64, _i64, _f, _i, _f, _p, _sz, _p]),
    "pamk_matmul_strided": (_i, [_p, _p, _p] + [_i64] * 16 + [_f, _i, _f, _i, _p, _sz, _p]),
    "pamk_logsumexp_fwd": (_i, [_p, _p, _i64, _i64, _f, _p, _sz, _p]),
    "pamk_logsumexp_bwd": (_i, [_p, _p, _p, _i64, _i64, _f, _i, _p, _sz, _p]),
    "pamk_ls_loss_fwd": (_i, [_p, _p, _p, _i64, _i64, _i, ctypes.c_longlong, _f, _p, _sz, _p]),
    "pamk_ls_loss_bwd": (_i, [_p, _p, _p, _p, _i64, _i64, _i, ctypes.c_longlong, _f, _i, _p, _sz, _p]),
    "pamk_cross_entropy_bwd": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _f, _f, _f, _i, ctypes.c_longlong, _f, _p, _sz, _p]),
    "pamk_adam_step": (_i, [_p, _p, _p, _p, _p, _i] + [_f] * 8 + [_p]),
    "pamk_issue_rate": (_i, [_i, _i, _i, _p, ctypes.POINTER(_f), ctypes.POINTER(ctypes.c_double), _p]),
}

_lib = None
_traced = None
_nvtx = os.environ.get("PAM_B200_NVTX", "") not in ("", "0")


class _Traced:
    """The library with every entry point that takes a stream wrapped in an NVTX range named after
    it, so that a timeline shows which library call a kernel belongs to (the reference's forks mark
    their steps with record_function scopes and emit_nvtx, fairseq_cli/train.py:569-571)."""

    def __init__(self, handle):
        self._handle = handle
        self._wrapped = {}

    def __getattr__(self, name):
        fn = getattr(self._handle, name)
        args = _SIGNATURES.get(name, (None, ()))[1]
        if not args or args[-1] is not _p:                 # no stream argument: nothing is launched
            return fn
        wrapped = self._wrapped.get(name)
        if wrapped is None:
            def wrapped(*a, _fn=fn, _name=name):
                torch.cuda.nvtx.range_push(_name)
                try:
                    return _fn(*a)
                finally:
                    torch.cuda.nvtx.range_pop()
            self._wrapped[name] = wrapped
        return wrapped


def set_nvtx(on):
    """Turns the NVTX ranges around the library's launches on or off (also: PAM_B200_NVTX=1)."""
    global _nvtx
    _nvtx = bool(on)


def lib():
    """The loaded library; raises if it was never built (``python -m pam_b200.build``)."""
    global _lib, _traced
    if _lib is not None and _nvtx:
        if _traced is None:
            _traced = _Traced(_lib)
        return _traced
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing. pam_b200 has no fallback path: build the CUDA kernels first "
                "with `python -m pam_b200.build` (needs nvcc).")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return lib() if _nvtx else _lib


def exported_names():
    return list(_SIGNATURES)


class PamKernelError(RuntimeError):
    pass


def check(status, what):
    if status != 0:
        handle = lib()
        msg = handle.pamk_status_string(status).decode()
        if status == -5:
            msg += f" [cudaError {handle.pamk_last_cuda_error()}]"
        raise PamKernelError(f"{what}: {msg}")


def require_cuda(*tensors):
    """All tensor operands must be fp32-convertible CUDA tensors on one device."""
    dev = None
    for t in tensors:
        if not isinstance(t, torch.Tensor):
            continue
        if not t.is_cuda:
            raise RuntimeError("pam_b200 runs on CUDA tensors only (there is no CPU path); got a "
                               f"{t.device.type} tensor")
        if dev is not None and t.device != dev:
            raise RuntimeError(f"operands on different devices: {dev} and {t.device}")
        dev = t.device
    if dev is None:
        raise RuntimeError("at least one operand must be a CUDA tensor")
    return dev


def stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream


import contextlib

_NO_GUARD = contextlib.nullcontext()


def device_guard(device):
    """Makes `device` current for the duration of a kernel launch (free when it already is)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)
