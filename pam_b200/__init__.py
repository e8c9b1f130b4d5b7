"""pam_b200 — piecewise affine multiplication (PAM) for NVIDIA B200.

A drop-in for the ``pam`` package of epfml/pam: the same functions (``mul div exp exp2 log log2
pow matmul bmm linear conv2d conv2d_group mean softmax logsumexp log_softmax layer_norm
cross_entropy``), modules (``Linear Conv2d LayerNorm``) and submodules (``pam_ops native pam_opt
pam_experimental cuda_bindings utils``), computed by hand-written sm_100a kernels behind the C ABI
of ``include/pam_b200.h``.  ``pam_b200.factories`` mirrors ``shared/modules/factories.py`` and
``pam_b200.optim.Adam`` the PAM Adam of the reference's fairseq fork.

``install_as_pam()`` registers this package under the reference's import names so that code
written against the reference (``import pam``, ``from shared.modules import factories``) runs
unchanged.
"""
import sys
import types

from . import pam_experimental, utils                      # noqa: F401
from . import cuda_bindings, native, pam_ops, pam_opt      # noqa: F401
from .pam_ops import *                                     # noqa: F401,F403
from .pam_opt import cross_entropy, cross_entropy_autograd  # noqa: F401
from .cuda_bindings import set_strict_k_order, strict_k_order  # noqa: F401
from ._lib import set_nvtx  # noqa: F401

__version__ = "0.1.0"


def install_as_pam():
    """Aliases ``pam`` (+ submodules) and ``shared.modules.factories`` to this package."""
    from . import factories, optim  # noqa: F401
    me = sys.modules[__name__]
    sys.modules.setdefault("pam", me)
    for sub in ("pam_ops", "pam_opt", "native", "cuda_bindings", "pam_experimental", "utils"):
        sys.modules.setdefault(f"pam.{sub}", sys.modules[f"{__name__}.{sub}"])
    shared = sys.modules.setdefault("shared", types.ModuleType("shared"))
    modules = sys.modules.setdefault("shared.modules", types.ModuleType("shared.modules"))
    shared.modules = modules
    modules.factories = factories
    sys.modules.setdefault("shared.modules.factories", factories)
    return me
