"""Generates tests/golden/full_batch_golden.npz: one forward + backward pass of each of the two
training workloads at the batch the benchmark runs them with (DeiT-tiny: 64 images of 224 x 224;
the 6+6 transformer: 128 sentence pairs of 32 tokens = 4096 tokens per side, vocabulary 10000),
evaluated by the REFERENCE's operator library on the CPU.

    python tests/golden/make_full_batch_golden.py [deit] [transformer]
        (run where the reference tree is mounted; about 10 and 20 minutes on 8 cores)

Same arrangement as make_step_golden.py: the graphs are pam_b200/steps.py, every PAM operation in them
is the reference's own pam_ops / cuda_bindings code, with the JIT-built extension replaced by a
stand-in that evaluates the reference's scalar device functions (pam/cuda_kernels.cu:15-136,
host-compiled as oracle/_ref/libpam_ref.so).

A full set of gradients would be 22 MB (DeiT) and 170 MB (transformer), so the fixture keeps, per
parameter, the first SAMPLE elements of up to ROWS rows spread evenly over its first dimension (all of
a 1-D parameter up to SAMPLE elements), next to the loss.  Inputs and parameters are not stored: the
test regenerates them from the same seeds.
"""
import os
import pathlib
import sys
import time

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

sys.path.insert(0, str(ROOT / "tests"))
from full_batch_cases import CASES, sample  # noqa: E402


def main(names):
    path = pathlib.Path(__file__).with_name("full_batch_golden.npz")
    out = dict(np.load(path)) if path.exists() else {}
    for name in names:
        params, loss_of = CASES[name]()
        leaves = {k: v.clone().requires_grad_() for k, v in params.items()}
        t0 = time.time()
        loss = loss_of(ref_pam, leaves)
        t1 = time.time()
        loss.backward()
        print(f"{name}: loss {float(loss):.6f}, forward {t1 - t0:.0f} s, backward {time.time() - t1:.0f} s", flush=True)
        out = {k: v for k, v in out.items() if not k.startswith(name + "/")}
        out[f"{name}/loss"] = loss.detach().numpy().reshape(1)
        for k, leaf in leaves.items():
            out[f"{name}/grad/{k}"] = sample(leaf.grad).numpy()
            out[f"{name}/grad_max/{k}"] = leaf.grad.abs().max().numpy().reshape(1)
        np.savez_compressed(path, **{k: np.ascontiguousarray(v) for k, v in out.items()})
        print(f"{len(out)} arrays -> {path} ({path.stat().st_size / 1024:.0f} KiB)", flush=True)


if __name__ == "__main__":
    main(sys.argv[1:] or list(CASES))
