"""Generates tests/golden/step_golden.npz: one training step of each of the two workloads in
pam_b200/steps.py (a DeiT and an encoder-decoder transformer, at toy sizes) evaluated by the
REFERENCE's operator library.

    python tests/golden/make_step_golden.py        (run where the reference tree is mounted)

The graph definitions are this repository's; every PAM operation in them is the reference's own
(pam/pam_ops.py front-ends over pam/cuda_bindings.py autograd functions), run on CPU tensors the way
tests/golden/make_golden.py runs them: the JIT-built extension is replaced by a stand-in that
evaluates the reference's scalar device functions (pam/cuda_kernels.cu:15-136, host-compiled as
oracle/_ref/libpam_ref.so), and pam_ops' `native` name is pointed at `cuda_bindings` so that CPU
tensors take the kernel path.  The optimizer update replays the PAM Adam rule
(submodules/fairseq/fairseq/optim/adam.py:226-252) with the reference's mul / div / pow.

Per workload the fixture holds the inputs' seed-derived tensors, the loss, every gradient, every
parameter after the update, and the loss of a second forward pass with the updated parameters.
"""
import math
import os
import pathlib
import sys

import numpy as np
import torch

ROOT = pathlib.Path(__file__).resolve().parents[2]
REF = pathlib.Path(os.environ.get("PAM_REFERENCE_ROOT", "/root/reference"))
sys.path.insert(0, str(ROOT))

from oracle import build as oracle_build  # noqa: E402
from oracle import pam_oracle  # noqa: E402

oracle_build.build_oracle()
assert oracle_build.build_ref() is not None, "reference tree not mounted"

import torch.utils.cpp_extension as cpp_ext  # noqa: E402

cpp_ext.load = lambda **kw: pam_oracle.CpuKernels("reference")
sys.path.insert(0, str(REF))
import pam as ref_pam  # noqa: E402  (the reference package)
from pam import cuda_bindings, pam_ops  # noqa: E402

pam_ops.native = cuda_bindings  # CPU tensors -> kernel path

from pam_b200 import steps  # noqa: E402

KW = dict(approx_bwd=True)
LR, BETAS, EPS, WD = 5e-4, (0.9, 0.98), 1e-8, 0.05
OUT = {}

DEIT = steps.DeitConfig(image=16, patch=8, dim=24, depth=2, heads=3, mlp=48, classes=10)
TRANSFORMER = steps.TransformerConfig(vocab=40, dim=16, ffn=32, heads=4, encoder_layers=2, decoder_layers=2)


def adam_update(p, grad, step=1):
    m = pam_ops.mul(torch.zeros_like(p), BETAS[0]) + pam_ops.mul(grad, 1 - BETAS[0])
    v = pam_ops.mul(torch.zeros_like(p), BETAS[1])
    v = v + pam_ops.mul(pam_ops.mul(grad, grad), 1 - BETAS[1])
    denom = pam_ops.pow(v, 0.5) + EPS
    step_size = LR * math.sqrt(1 - BETAS[1] ** step) / (1 - BETAS[0] ** step)
    p = p - pam_ops.mul(p, WD * LR)
    return p - pam_ops.mul(pam_ops.div(m, denom), step_size)


def record(tag, params, loss_fn):
    leaves = {k: v.clone().requires_grad_() for k, v in params.items()}
    loss = loss_fn(leaves)
    loss.backward()
    OUT[f"{tag}/loss"] = loss.detach().numpy().reshape(1)
    updated = {}
    for k, leaf in leaves.items():
        OUT[f"{tag}/grad/{k}"] = leaf.grad.numpy()
        with torch.no_grad():
            updated[k] = adam_update(leaf.detach(), leaf.grad)
        OUT[f"{tag}/updated/{k}"] = updated[k].numpy()
    with torch.no_grad():
        OUT[f"{tag}/loss_after"] = loss_fn(updated).numpy().reshape(1)


g = torch.Generator().manual_seed(4)
params = steps.deit_params(DEIT, g)
images = torch.randn(3, DEIT.channels, DEIT.image, DEIT.image, generator=g)
labels = torch.randint(0, DEIT.classes, (3,), generator=g)
record("deit", params, lambda p: steps.deit_loss(ref_pam, p, images, labels, DEIT, KW))

g = torch.Generator().manual_seed(3)
params = steps.transformer_params(TRANSFORMER, g)
src, prev_out, target = steps.transformer_batch(TRANSFORMER, g, sentences=3, length=6)
record("transformer", params, lambda p: steps.transformer_loss(ref_pam, p, src, prev_out, target, TRANSFORMER, KW))

path = pathlib.Path(__file__).with_name("step_golden.npz")
np.savez_compressed(path, **{k: np.ascontiguousarray(v) for k, v in OUT.items()})
print(f"{len(OUT)} arrays -> {path} ({path.stat().st_size / 1024:.0f} KiB)")
