"""Cross entropy with a PAM backward — the counterpart of the reference's ``pam/pam_opt.py``."""
import torch


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
