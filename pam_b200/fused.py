"""Fused row kernels (layer normalisation, softmax) and the fused PAM Adam update.

Each fused op computes exactly the chain of PAM primitives that the reference runs as separate
launches from Python, rounding at the same points, in one pass over the data.  ``*_supported``
tells the operator library whether a call can take the fused route; otherwise it composes the
primitives one kernel at a time (still on the GPU).
"""
import math

import torch

from . import _lib

# Set to False to force the one-kernel-per-primitive composition everywhere (used by tests to
# compare the two routes).
enabled = True


def _offset(offset):
    return 1.0 if offset is None else float(offset)


def _ptr(t):
    return t.data_ptr() if t is not None else None


def _workspace(device, nbytes):
    from .cuda_bindings import _workspace as ws
    return ws(device, nbytes)


# ---- layer normalisation -------------------------------------------------------------------------

def _uniform(approx_bwd):
    """The fused kernels take one approx_bwd flag; a (first, second) pair must agree."""
    return isinstance(approx_bwd, bool) or len(set(approx_bwd)) == 1


def layer_norm_supported(x, normalized_shape, weight, bias, approx_bwd=False):
    if not (enabled and isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float32):
        return False
    if not _uniform(approx_bwd):
        return False
    width = math.prod(normalized_shape)
    if width > 1024 or x.numel() == 0:
        return False
    for p in (weight, bias):
        if p is not None and not (p.is_cuda and p.dtype == torch.float32 and p.numel() == width):
            return False
    return True


class _LayerNorm(torch.autograd.Function):
    """With the approximate backward (and a backward pass to come) the forward pass also keeps eight
    scalars per row, and the backward pass works from them instead of recomputing the row statistics."""

    @staticmethod
    def forward(ctx, x, weight, bias, width, eps, offset, approx, keep):
        rows2d = x.reshape(-1, width).contiguous()
        w = weight.contiguous().view(-1) if weight is not None else None
        b = bias.contiguous().view(-1) if bias is not None else None
        y = torch.empty_like(rows2d)
        dev = x.device
        handle = _lib.lib()
        stats = None
        with _lib.device_guard(dev):
            if approx and keep:
                stats = torch.empty(rows2d.shape[0], handle.pamk_layer_norm_stats_per_row(), dtype=torch.float32, device=dev)
                status = handle.pamk_layer_norm_fwd_save(rows2d.data_ptr(), _ptr(w), _ptr(b), y.data_ptr(), stats.data_ptr(),
                                                         rows2d.shape[0], width, eps, offset, _lib.stream_ptr(dev))
            else:
                status = handle.pamk_layer_norm_fwd(rows2d.data_ptr(), _ptr(w), _ptr(b), y.data_ptr(),
                                                    rows2d.shape[0], width, eps, offset, _lib.stream_ptr(dev))
        _lib.check(status, "pamk_layer_norm_fwd")
        ctx.save_for_backward(rows2d, w, stats)
        ctx.cfg = (width, eps, offset, approx, bias is not None, x.shape,
                   weight.shape if weight is not None else None, bias.shape if bias is not None else None)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, g):
        rows2d, w, stats = ctx.saved_tensors
        width, eps, offset, approx, has_bias, x_shape, w_shape, b_shape = ctx.cfg
        dev = rows2d.device
        g2 = g.reshape(-1, width).contiguous()
        dx = torch.empty_like(rows2d)
        need_w = w is not None and ctx.needs_input_grad[1]
        need_b = has_bias and ctx.needs_input_grad[2]
        dw = torch.empty(width, dtype=torch.float32, device=dev) if need_w else None
        db = torch.empty(width, dtype=torch.float32, device=dev) if need_b else None
        handle = _lib.lib()
        ws_bytes = handle.pamk_layer_norm_bwd_workspace_bytes(rows2d.shape[0], width) if (need_w or need_b) else 0
        ws = _workspace(dev, ws_bytes) if ws_bytes else None
        with _lib.device_guard(dev):
            if stats is not None:
                status = handle.pamk_layer_norm_bwd_saved(rows2d.data_ptr(), _ptr(w), g2.data_ptr(), stats.data_ptr(),
                                                          dx.data_ptr(), _ptr(dw), _ptr(db), rows2d.shape[0], width,
                                                          offset, _ptr(ws), ws_bytes, _lib.stream_ptr(dev))
            else:
                status = handle.pamk_layer_norm_bwd(rows2d.data_ptr(), _ptr(w), g2.data_ptr(), dx.data_ptr(), _ptr(dw),
                                                    _ptr(db), rows2d.shape[0], width, eps, offset, int(bool(approx)),
                                                    _ptr(ws), ws_bytes, _lib.stream_ptr(dev))
        _lib.check(status, "pamk_layer_norm_bwd")
        return (dx.view(x_shape), dw.view(w_shape) if need_w else None, db.view(b_shape) if need_b else None,
                None, None, None, None, None)


def layer_norm(x, normalized_shape, weight, bias, eps, *, offset=None, approx_bwd=False):
    if not isinstance(approx_bwd, bool):
        approx_bwd = bool(approx_bwd[0])
    keep = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (x, weight, bias))
    return _LayerNorm.apply(x, weight, bias, math.prod(normalized_shape), float(eps), _offset(offset), approx_bwd, keep)


# ---- softmax ---------------------------------------------------------------------------------------

_MAX_ROW = 12288


def _last_dim(x, dim):
    return isinstance(dim, int) and x.dim() > 0 and dim in (-1, x.dim() - 1)


def softmax_supported(x, dim, approx_bwd=False):
    return (enabled and isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float32 and
            _last_dim(x, dim) and 0 < x.shape[-1] <= _MAX_ROW and x.numel() > 0 and _uniform(approx_bwd))


def _rows(handle, name, x2, extra, out, offset, approx=None):
    dev = x2.device
    rows, length = x2.shape
    ws_bytes = handle.pamk_softmax_workspace_bytes(rows, length)
    ws = _workspace(dev, ws_bytes)
    args = [x2.data_ptr()] + [t.data_ptr() for t in extra] + [out.data_ptr(), rows, length, offset]
    if approx is not None:
        args.append(int(bool(approx)))
    with _lib.device_guard(dev):
        status = getattr(handle, name)(*args, ws.data_ptr(), ws_bytes, _lib.stream_ptr(dev))
    _lib.check(status, name)
    return out


def _softmax_forward_saving(x2, offset):
    """Softmax of the rows of x2 plus the exponentials the approximate backward pass works from."""
    y, e = torch.empty_like(x2), torch.empty_like(x2)
    _rows(_lib.lib(), "pamk_softmax_fwd_save", x2, [y], e, offset)
    return y, e


def _softmax_backward_saved(e, g2, offset, post_scale=None):
    dev = e.device
    dx = torch.empty_like(e)
    rows, length = e.shape
    with _lib.device_guard(dev):
        status = _lib.lib().pamk_softmax_bwd_saved(e.data_ptr(), g2.data_ptr(), dx.data_ptr(), rows, length, offset,
                                                   int(post_scale is not None), float(post_scale or 0.0),
                                                   _lib.stream_ptr(dev))
    _lib.check(status, "pamk_softmax_bwd_saved")
    return dx


class _Softmax(torch.autograd.Function):
    """With the approximate backward the forward pass keeps its exponentials instead of its input: the
    backward pass then needs neither the maximum pass nor the exp2 chain (same values either way)."""

    @staticmethod
    def forward(ctx, x, offset, approx, keep):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        ctx.cfg = (offset, approx, x.shape)
        if approx and keep:
            y, e = _softmax_forward_saving(x2, offset)
            ctx.save_for_backward(e)
            return y.view(x.shape)
        ctx.save_for_backward(x2)
        return _rows(_lib.lib(), "pamk_softmax_fwd", x2, [], torch.empty_like(x2), offset).view(x.shape)

    @staticmethod
    def backward(ctx, g):
        (saved,) = ctx.saved_tensors
        offset, approx, shape = ctx.cfg
        g2 = g.reshape(saved.shape).contiguous()
        if approx:
            return _softmax_backward_saved(saved, g2, offset).view(shape), None, None, None
        dx = _rows(_lib.lib(), "pamk_softmax_bwd", saved, [g2], torch.empty_like(saved), offset, approx)
        return dx.view(shape), None, None, None


class _LogSumExp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, offset, approx):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        ctx.save_for_backward(x2)
        ctx.cfg = (offset, approx, x.shape)
        out = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        return _rows(_lib.lib(), "pamk_logsumexp_fwd", x2, [], out, offset).view(x.shape[:-1])

    @staticmethod
    def backward(ctx, g):
        (x2,) = ctx.saved_tensors
        offset, approx, shape = ctx.cfg
        g1 = g.reshape(-1).contiguous()
        dx = _rows(_lib.lib(), "pamk_logsumexp_bwd", x2, [g1], torch.empty_like(x2), offset, approx)
        return dx.view(shape), None, None


def _flag(approx_bwd):
    return approx_bwd if isinstance(approx_bwd, bool) else bool(approx_bwd[0])


def softmax(x, dim, *, offset=None, approx_bwd=False):
    # (the exponentials are only worth writing when a backward pass can follow)
    return _Softmax.apply(x, _offset(offset), _flag(approx_bwd), torch.is_grad_enabled() and x.requires_grad)


def logsumexp(x, dim, keepdim=False, *, offset=None, approx_bwd=False):
    out = _LogSumExp.apply(x, _offset(offset), _flag(approx_bwd))
    return out.unsqueeze(-1) if keepdim else out


# ---- attention over a fused q/k/v projection ------------------------------------------------------------

def attention_supported(qkv, num_heads, approx_bwd=False):
    """The strided route below needs fp32 CUDA input [B, N, 3*C] with C divisible by the heads, rows that
    the softmax kernel can hold, at most 65535 (batch, head) pairs and the approximate backward for every
    operand (the exact-gradient products take the forward output as a third operand)."""
    if not (enabled and isinstance(qkv, torch.Tensor) and qkv.is_cuda and qkv.dtype == torch.float32):
        return False
    if qkv.dim() != 3 or qkv.numel() == 0 or qkv.shape[-1] % (3 * num_heads):
        return False
    approx = (approx_bwd,) if isinstance(approx_bwd, bool) else tuple(approx_bwd)
    return all(approx) and qkv.shape[1] <= _MAX_ROW and qkv.shape[0] * num_heads <= 65535


def _strided_product(dev, a_ptr, b_ptr, c_ptr, outer, inner, M, N, K, sa, sb, sc, offset, post_scale=None):
    """One pamk_matmul_strided call with the split the plain product of the same shape would get."""
    handle = _lib.lib()
    split = handle.pamk_matmul_auto_split(outer * inner, M, N, K)
    ws_ptr, ws_bytes = None, 0
    if split > 1:
        ws_bytes = handle.pamk_matmul_workspace_bytes(outer * inner, M, N, split)
        ws_ptr = _workspace(dev, ws_bytes).data_ptr()
    with _lib.device_guard(dev):
        status = handle.pamk_matmul_strided(a_ptr, b_ptr, c_ptr, outer, inner, M, N, K, *sa, *sb, *sc, offset,
                                            int(post_scale is not None), float(post_scale or 0.0), split,
                                            ws_ptr, ws_bytes, _lib.stream_ptr(dev))
    _lib.check(status, "pamk_matmul_strided")


class _AttentionQKV(torch.autograd.Function):
    """softmax(pam(q k^T, scale)) v on the heads of a fused projection, reading q, k, v where the projection
    wrote them ([B, N, 3, heads, head_dim]) and writing the context token-major ([B, N, C]): the products,
    the PAM scaling (in the score product's epilogue), the softmax and every gradient product have the
    shapes, split-K plans and arithmetic of the chain bmm -> mul -> softmax -> bmm on flattened copies
    (timm vision_transformer.py:72-93 in the fork), so the values are the same bit for bit; what is left out
    are the copies around them and the two passes of the scaling over the [B*heads, N, N] scores."""

    @staticmethod
    def forward(ctx, qkv, heads, scale, offset):
        qkv = qkv.contiguous()
        B, N, C3 = qkv.shape
        C = C3 // 3
        hd = C // heads
        dev = qkv.device
        base = qkv.data_ptr()
        q_ptr, k_ptr, v_ptr = base, base + 4 * C, base + 8 * C
        scores = torch.empty(B * heads, N, N, dtype=torch.float32, device=dev)
        # scores = pam(q k^T, scale): q rows and k rows are 3C apart, heads hd apart
        _strided_product(dev, q_ptr, k_ptr, scores.data_ptr(), B, heads, N, N, hd,
                         (N * C3, hd, C3, 1), (N * C3, hd, 1, C3), (heads * N * N, N * N, N), offset, post_scale=scale)
        probs, expo = _softmax_forward_saving(scores.view(-1, N), offset)
        out = torch.empty(B, N, C, dtype=torch.float32, device=dev)
        # context[b, i, h, :] = probs[b, h, i, :] v[b, :, h, :]
        _strided_product(dev, probs.data_ptr(), v_ptr, out.data_ptr(), B, heads, N, hd, N,
                         (heads * N * N, N * N, N, 1), (N * C3, hd, C3, 1), (N * C, hd, C), offset)
        ctx.save_for_backward(qkv, expo, probs)
        ctx.cfg = (heads, scale, offset)
        return out

    @staticmethod
    def backward(ctx, g):
        qkv, expo, probs = ctx.saved_tensors
        heads, scale, offset = ctx.cfg
        B, N, C3 = qkv.shape
        C = C3 // 3
        hd = C // heads
        dev = qkv.device
        g = g.contiguous()
        base = qkv.data_ptr()
        q_ptr, k_ptr, v_ptr = base, base + 4 * C, base + 8 * C
        dqkv = torch.empty_like(qkv)
        dq_ptr, dv_ptr = dqkv.data_ptr(), dqkv.data_ptr() + 8 * C
        s_probs, s_ctx = (heads * N * N, N * N, N, 1), (N * C, hd, C, 1)
        # d probs = d context v^T
        dprobs = torch.empty(B * heads, N, N, dtype=torch.float32, device=dev)
        _strided_product(dev, g.data_ptr(), v_ptr, dprobs.data_ptr(), B, heads, N, N, hd,
                         s_ctx, (N * C3, hd, 1, C3), (heads * N * N, N * N, N), offset)
        # d v = probs^T d context, written where v's gradient lives in d qkv
        _strided_product(dev, probs.data_ptr(), g.data_ptr(), dv_ptr, B, heads, N, hd, N,
                         (heads * N * N, N * N, 1, N), (N * C, hd, C, 1), (N * C3, hd, C3), offset)
        # d scores = pam(softmax backward, scale), from the exponentials the forward pass kept
        dscores = _softmax_backward_saved(expo, dprobs.view(-1, N), offset, post_scale=scale)
        # d q = d scores k
        _strided_product(dev, dscores.data_ptr(), k_ptr, dq_ptr, B, heads, N, hd, N,
                         s_probs, (N * C3, hd, C3, 1), (N * C3, hd, C3), offset)
        # d (k^T) = q^T d scores as the chain computes it ([head_dim, N] per head), then into k's slot
        dkt = torch.empty(B, heads, hd, N, dtype=torch.float32, device=dev)
        _strided_product(dev, q_ptr, dscores.data_ptr(), dkt.data_ptr(), B, heads, hd, N, N,
                         (N * C3, hd, 1, C3), (heads * N * N, N * N, N, 1), (heads * hd * N, hd * N, N), offset)
        dqkv.view(B, N, 3, heads, hd)[:, :, 1].copy_(dkt.permute(0, 3, 1, 2))
        return dqkv, None, None, None


def attention_heads_supported(q, k, v, num_heads, mask=None, approx_bwd=False):
    """Like attention_supported, for separate query / key / value projections ([B, T, d], [B, S, d], [B, S, d])
    and an optional additive mask that needs no gradient."""
    for t in (q, k, v):
        if not (enabled and isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.float32 and t.dim() == 3):
            return False
    if q.numel() == 0 or k.numel() == 0 or k.shape != v.shape or q.shape[0] != k.shape[0] or q.shape[2] != k.shape[2]:
        return False
    if q.shape[2] % num_heads or q.shape[0] * num_heads > 65535 or k.shape[1] > _MAX_ROW:
        return False
    if mask is not None and not (isinstance(mask, torch.Tensor) and mask.is_cuda and mask.dtype == torch.float32
                                 and not mask.requires_grad):
        return False
    approx = (approx_bwd,) if isinstance(approx_bwd, bool) else tuple(approx_bwd)
    return all(approx)


class _AttentionHeads(torch.autograd.Function):
    """softmax(q k^T + mask) v per head for separate projections q [B, T, d], k, v [B, S, d] (the explicit
    branch of the fairseq fork's attention, fairseq/modules/multihead_attention.py:618-783, which splits the
    heads into copies, multiplies, adds the mask, takes the softmax, multiplies and merges the heads through
    another copy).  As in _AttentionQKV the heads are strided views of the projections, the context is written
    token-major, every product has the shape and split-K plan of the chain's, and the values are the chain's
    bit for bit."""

    @staticmethod
    def forward(ctx, q, k, v, mask, heads, offset):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        B, T, d = q.shape
        S = k.shape[1]
        hd = d // heads
        dev = q.device
        scores = torch.empty(B * heads, T, S, dtype=torch.float32, device=dev)
        _strided_product(dev, q.data_ptr(), k.data_ptr(), scores.data_ptr(), B, heads, T, S, hd,
                         (T * d, hd, d, 1), (S * d, hd, 1, d), (heads * T * S, T * S, S), offset)
        if mask is not None:
            scores.add_(mask)
        probs, expo = _softmax_forward_saving(scores.view(-1, S), offset)
        out = torch.empty(B, T, d, dtype=torch.float32, device=dev)
        _strided_product(dev, probs.data_ptr(), v.data_ptr(), out.data_ptr(), B, heads, T, hd, S,
                         (heads * T * S, T * S, S, 1), (S * d, hd, d, 1), (T * d, hd, d), offset)
        ctx.save_for_backward(q, k, v, expo, probs)
        ctx.cfg = (heads, offset)
        return out

    @staticmethod
    def backward(ctx, g):
        q, k, v, expo, probs = ctx.saved_tensors
        heads, offset = ctx.cfg
        B, T, d = q.shape
        S = k.shape[1]
        hd = d // heads
        dev = q.device
        g = g.contiguous()
        s_scores, s_q, s_kv = (heads * T * S, T * S, S, 1), (T * d, hd, d, 1), (S * d, hd, d, 1)
        # d probs = d context v^T
        dprobs = torch.empty(B * heads, T, S, dtype=torch.float32, device=dev)
        _strided_product(dev, g.data_ptr(), v.data_ptr(), dprobs.data_ptr(), B, heads, T, S, hd,
                         s_q, (S * d, hd, 1, d), (heads * T * S, T * S, S), offset)
        # d v = probs^T d context
        dv = torch.empty_like(v)
        _strided_product(dev, probs.data_ptr(), g.data_ptr(), dv.data_ptr(), B, heads, S, hd, T,
                         (heads * T * S, T * S, 1, S), s_q, (S * d, hd, d), offset)
        # d scores (the mask is a constant)
        dscores = _softmax_backward_saved(expo, dprobs.view(-1, S), offset)
        # d q = d scores k
        dq = torch.empty_like(q)
        _strided_product(dev, dscores.data_ptr(), k.data_ptr(), dq.data_ptr(), B, heads, T, hd, S,
                         s_scores, s_kv, (T * d, hd, d), offset)
        # d (k^T) = q^T d scores as the chain computes it ([head_dim, S] per head), then transposed into d k
        dkt = torch.empty(B, heads, hd, S, dtype=torch.float32, device=dev)
        _strided_product(dev, q.data_ptr(), dscores.data_ptr(), dkt.data_ptr(), B, heads, hd, S, T,
                         (T * d, hd, 1, d), s_scores, (heads * hd * S, hd * S, S), offset)
        dk = torch.empty_like(k)
        dk.view(B, S, heads, hd).copy_(dkt.permute(0, 3, 1, 2))
        return dq, dk, dv, None, None, None


def attention_heads(q, k, v, num_heads, mask=None, *, offset=None):
    return _AttentionHeads.apply(q, k, v, mask, int(num_heads), _offset(offset))


def attention_qkv(qkv, num_heads, scale, *, offset=None):
    return _AttentionQKV.apply(qkv, int(num_heads), float(scale), _offset(offset))


# ---- loss kernels ---------------------------------------------------------------------------------------

def loss_supported(logits, target):
    return (enabled and isinstance(logits, torch.Tensor) and logits.is_cuda and logits.dtype == torch.float32 and
            logits.dim() == 2 and 0 < logits.shape[-1] <= _MAX_ROW and logits.shape[0] > 0 and
            isinstance(target, torch.Tensor) and target.device == logits.device and target.dtype == torch.int64 and
            target.numel() == logits.shape[0])


def _loss_call(name, logits, args):
    dev = logits.device
    handle = _lib.lib()
    rows, length = logits.shape
    ws_bytes = handle.pamk_softmax_workspace_bytes(rows, length)
    ws = _workspace(dev, ws_bytes)
    with _lib.device_guard(dev):
        status = getattr(handle, name)(*args, ws.data_ptr(), ws_bytes, _lib.stream_ptr(dev))
    _lib.check(status, name)


class _LabelSmoothedSums(torch.autograd.Function):
    """(sum of -lprobs[target], sum of -lprobs over all classes) of the PAM log-softmax of `logits`,
    from the logits in one row pass; rows whose target is `ignore_index` contribute nothing."""

    @staticmethod
    def forward(ctx, logits, target, ignore_index, offset, approx):
        x2 = logits.contiguous()
        tgt = target.reshape(-1).contiguous()
        rows, length = x2.shape
        out = torch.empty(rows, 3, dtype=torch.float32, device=x2.device)
        has_ignore = ignore_index is not None
        _loss_call("pamk_ls_loss_fwd", x2, [x2.data_ptr(), tgt.data_ptr(), out.data_ptr(), rows, length,
                                            int(has_ignore), int(ignore_index or 0), offset])
        ctx.save_for_backward(x2, tgt)
        ctx.cfg = (ignore_index, offset, approx)
        return out[:, 1].sum(), out[:, 2].sum()

    @staticmethod
    def backward(ctx, g_nll, g_smooth):
        x2, tgt = ctx.saved_tensors
        ignore_index, offset, approx = ctx.cfg
        rows, length = x2.shape
        grads = torch.stack([g_nll.reshape(()).float(), g_smooth.reshape(()).float()]).contiguous()
        dx = torch.empty_like(x2)
        has_ignore = ignore_index is not None
        _loss_call("pamk_ls_loss_bwd", x2, [x2.data_ptr(), tgt.data_ptr(), grads.data_ptr(), dx.data_ptr(), rows, length,
                                            int(has_ignore), int(ignore_index or 0), offset, int(bool(approx))])
        return dx, None, None, None, None


def label_smoothed_sums(logits, target, ignore_index=None, *, offset=None, approx_bwd=False):
    return _LabelSmoothedSums.apply(logits, target, ignore_index, _offset(offset), _flag(approx_bwd))


def cross_entropy_grad(logits, target, weight, grad_out, *, hot, cold, mean_rows, ignore_index=None, offset=None):
    """The gradient of pam_opt.cross_entropy with respect to the logits in one launch (see
    pamk_cross_entropy_bwd in the C header); `grad_out` is the incoming 0-d gradient tensor."""
    x2 = logits.contiguous()
    tgt = target.reshape(-1).contiguous()
    rows, length = x2.shape
    dx = torch.empty_like(x2)
    w = None if weight is None else weight.detach().float().contiguous()
    g = grad_out.detach().reshape(1).float().contiguous()
    has_ignore = ignore_index is not None
    _loss_call("pamk_cross_entropy_bwd", x2, [x2.data_ptr(), tgt.data_ptr(), None if w is None else w.data_ptr(), g.data_ptr(),
                                              dx.data_ptr(), rows, length, float(hot), float(cold), float(mean_rows),
                                              int(has_ignore), int(ignore_index or 0), _offset(offset)])
    return dx


# ---- linear layer with bias ----------------------------------------------------------------------------

def linear_bias_supported(X2, W, bias):
    """The bias can ride in the product's epilogue when it is a plain fp32 vector of the output width
    on the operands' device."""
    return (enabled and isinstance(bias, torch.Tensor) and isinstance(X2, torch.Tensor) and isinstance(W, torch.Tensor)
            and X2.is_cuda and bias.device == X2.device and W.device == X2.device
            and bias.dtype == torch.float32 and bias.dim() == 1
            and W.dim() == 2 and bias.shape[0] == W.shape[0] and bias.is_contiguous()
            and X2.dtype == torch.float32 and W.dtype == torch.float32)


# ---- Adam --------------------------------------------------------------------------------------------

def adam_supported(p, grad):
    return (enabled and p.is_cuda and p.dtype == torch.float32 and grad.dtype == torch.float32 and
            p.is_contiguous() and grad.is_contiguous() and grad.device == p.device)


def adam_step(tensors, *, beta1, beta2, eps, step_size, decay, offset=None):
    """One PAM Adam update, in place, of every (param, grad, exp_avg, exp_avg_sq) in `tensors`
    (all fp32, contiguous, on one CUDA device) with shared scalars.  The scalars arrive as Python
    doubles and are rounded to fp32 here, once, like the reference's scalar-to-tensor promotion."""
    import ctypes
    if not tensors:
        return
    dev = tensors[0][0].device
    count = len(tensors)
    ptrs = [(ctypes.c_void_p * count)(*[t[k].data_ptr() for t in tensors]) for k in range(4)]
    sizes = (ctypes.c_int64 * count)(*[t[0].numel() for t in tensors])
    with _lib.device_guard(dev):
        status = _lib.lib().pamk_adam_step(*ptrs, sizes, count, beta1, 1 - beta1, beta2, 1 - beta2, eps,
                                           decay, step_size, _offset(offset), _lib.stream_ptr(dev))
    _lib.check(status, "pamk_adam_step")
