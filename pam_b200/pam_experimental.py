"""Base-2 softmax family in ordinary floating point (no PAM arithmetic): the functions behind the
reference's ``standard2`` function dictionary (pam/pam_experimental.py).  They share the PAM
softmax's structure — a whole-tensor ``floor(max)`` shift and ``exp2`` — with exact arithmetic."""
import torch


def _shifted_exp2(x, dtype):
    if dtype is not None:
        x = x.to(dtype=dtype)
    with torch.no_grad():
        shift = torch.floor(torch.max(x))
    return x, shift, torch.exp2(x - shift)


def torch_softmax2(x, dim=None, dtype=None):
    _, _, e = _shifted_exp2(x, dtype)
    return e / torch.sum(e, dim=dim, keepdim=True)


def torch_logsumexp2(x, dim=None, keepdim=None, dtype=None):
    _, shift, e = _shifted_exp2(x, dtype)
    return torch.log2(torch.sum(e, dim=dim, keepdim=keepdim)) + shift


def torch_log_softmax2(x, dim=None, dtype=None):
    if dtype is not None:
        x = x.to(dtype=dtype)
    return x - torch_logsumexp2(x, dim=dim, keepdim=True)


def torch_cross_entropy2(x, target, weight=None, ignore_index=-100, reduction="mean", label_smoothing=0.0):
    log_prob = x - torch_logsumexp2(x, dim=-1)
    keep = None
    if ignore_index is not None:
        keep = ~target.eq(ignore_index)
        target = torch.where(keep, target, torch.zeros_like(target))
    prob = torch.nn.functional.one_hot(target, num_classes=x.shape[-1]).float()
    if label_smoothing:
        prob = prob * (1 - label_smoothing) + label_smoothing / x.shape[-1]
    terms = -log_prob * prob
    if keep is not None:
        terms = terms * keep.view(-1, 1)
    if weight is not None:
        terms = terms * weight.view(-1, 1)
    loss = torch.sum(terms, dim=-1)
    if reduction == "mean":
        return torch.mean(loss)
    if reduction == "sum":
        return torch.sum(loss)
    if reduction is not None:
        raise ValueError("Unknown reduction")
    return loss
