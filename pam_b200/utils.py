"""Scalar / tensor helpers with the semantics of the reference's ``pam/utils.py``."""
import torch


def to_tensor(*values, device=None):
    """Python numbers become fp32 0-d tensors on the device of the tensor operands
    (pam/utils.py:3-17); tensors pass through unchanged."""
    for v in values:
        if isinstance(v, torch.Tensor):
            assert device is None or device == v.device, f"Mismatching devices {device=}, {v.device=}"
            device = v.device
    return [torch.tensor(v, device=device, dtype=torch.float32) if isinstance(v, (int, float)) else v
            for v in values]


def broadcast_tensors(*tensors):
    return torch.broadcast_tensors(*to_tensor(*tensors))


def demote_tensor(out_value, in_values):
    """A call whose inputs were all Python numbers returns a Python float (pam/utils.py:23-27)."""
    if all(isinstance(v, (float, int)) for v in in_values):
        return out_value.item()
    return out_value


def is_number(v):
    return isinstance(v, (int, float)) and not isinstance(v, bool)
