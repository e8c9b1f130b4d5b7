"""Cross entropy with a PAM backward — the counterpart of the reference's ``pam/pam_opt.py`` — and the
label-smoothed loss of the reference's fairseq criterion computed straight from the logits."""
import torch

from . import fused, pam_ops


def _pam_binding(ops, names):
    """If the entries `names` of an operator dictionary are this package's PAM functions, bound (by the
    factories' dict-form configuration) to one common set of keyword arguments, those arguments; else
    None.  Lets a chain of dictionary calls be replaced by one fused kernel without changing results."""
    common = None
    for name in names:
        op = ops.get(name)
        func, kwargs = getattr(op, "pam_function", op), getattr(op, "pam_kwargs", {})
        if func is not getattr(pam_ops, name):
            return None
        kwargs = {k: v for k, v in kwargs.items() if k in ("offset", "approx_bwd")}
        if common is not None and kwargs != common:
            return None
        common = kwargs
    return common


class cross_entropy_autograd(torch.autograd.Function):
    """Forward returns the ordinary loss value (for comparison with standard training); the
    gradient is (softmax(X) - target distribution), scaled by class weights, the batch mean and
    the incoming gradient, all through the caller's ``op_dict`` (pam/pam_opt.py:6-51)."""

    @staticmethod
    def forward(ctx, X, Y, weight=None, ignore_index=None, reduction="mean", label_smoothing=0.0, op_dict=None):
        assert op_dict is not None, "OP dict must be explicitly specified"
        ctx.save_for_backward(X, Y, weight)
        ctx.cfg = (ignore_index, reduction, label_smoothing, op_dict)
        return torch.nn.functional.cross_entropy(
            input=X, target=Y, weight=weight, ignore_index=ignore_index,
            reduction=reduction, label_smoothing=label_smoothing)

    @staticmethod
    def backward(ctx, delta_output):
        X, Y, weight = ctx.saved_tensors
        ignore_index, reduction, label_smoothing, ops = ctx.cfg
        classes = X.shape[-1]
        bound = _pam_binding(ops, ("softmax", "mul", "div"))
        if bound is not None and X.dim() == 2 and fused.loss_supported(X, Y) and delta_output.numel() == 1:
            # the whole chain below in one row kernel (same values: the target distribution's two
            # probabilities are formed here in fp32 exactly as the tensor expressions below form them)
            one, zero = torch.ones((), dtype=torch.float32), torch.zeros((), dtype=torch.float32)
            hot, cold = one, zero
            if label_smoothing:
                hot, cold = one * (1 - label_smoothing), zero * (1 - label_smoothing)
                hot, cold = hot + (label_smoothing / classes) * one, cold + (label_smoothing / classes) * one
            delta = fused.cross_entropy_grad(X, Y, weight, delta_output, hot=float(hot), cold=float(cold),
                                             mean_rows=X.shape[0] if reduction == "mean" else 0,
                                             ignore_index=ignore_index, offset=bound.get("offset"))
            return (delta,) + (None,) * 6
        prob = ops["softmax"](X, dim=-1)
        ignored = None
        if ignore_index is not None:
            ignored = Y.eq(ignore_index)
            Y = Y.masked_fill(ignored, 0)          # any valid class; the row is zeroed below
        target = torch.nn.functional.one_hot(Y, num_classes=classes).float()
        if label_smoothing:
            target = target * (1 - label_smoothing)
            target = target + (label_smoothing / classes) * torch.ones_like(target)
        delta = prob - target
        if weight is not None:
            delta = ops["mul"](delta, weight[Y].view(-1, 1))
        if ignored is not None:
            delta = delta * (~ignored.view(-1, 1))
        if reduction == "mean":
            delta = ops["div"](delta, X.shape[0])
        delta = ops["mul"](delta, delta_output.view(-1, 1))
        return (delta,) + (None,) * 6


def cross_entropy(X, Y, weight=None, ignore_index=None, reduction="mean", label_smoothing=0.0, *, op_dict=None):
    return cross_entropy_autograd.apply(X, Y, weight, ignore_index, reduction, label_smoothing, op_dict)


def label_smoothed_nll_loss(logits, target, epsilon, ignore_index=None, *, op_dict=None):
    """fairseq's ``label_smoothed_nll_loss`` (criterions/label_smoothed_cross_entropy.py:36-54, with
    ``reduce=True``) taken from the logits instead of from log-probabilities: returns (loss, nll_loss)
    where lprobs = op_dict['log_softmax'](logits).  With a PAM operator dictionary the log-softmax, the
    gather and the two sums run in one row kernel forward and one backward; otherwise the reference's
    sequence of dictionary calls runs as it stands.  logits [rows, classes], target [rows]."""
    assert op_dict is not None, "OP dict must be explicitly specified"
    classes = logits.shape[-1]
    bound = _pam_binding(op_dict, ("log_softmax", "mul", "div"))
    if bound is not None and fused.loss_supported(logits, target.reshape(-1)):
        nll, smooth = fused.label_smoothed_sums(logits, target.reshape(-1), ignore_index, offset=bound.get("offset"),
                                                approx_bwd=bound.get("approx_bwd", False))
    else:
        lprobs = op_dict["log_softmax"](logits, dim=-1)
        tgt = target.reshape(-1, 1)
        nll, smooth = -lprobs.gather(dim=-1, index=tgt), -lprobs.sum(dim=-1, keepdim=True)
        if ignore_index is not None:
            pad = tgt.eq(ignore_index)
            nll, smooth = nll.masked_fill(pad, 0.0), smooth.masked_fill(pad, 0.0)
        nll, smooth = nll.sum(), smooth.sum()
    eps_i = op_dict["div"](epsilon, classes - 1)
    return op_dict["mul"](1.0 - epsilon - eps_i, nll) + op_dict["mul"](eps_i, smooth), nll
