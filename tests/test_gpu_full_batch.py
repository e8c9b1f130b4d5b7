"""The two training workloads at the benchmark's batch (DeiT-tiny: 64 images; transformer: 4096 tokens
per side) against the fixture that the reference's own operator library produced for the same seeds
(tests/golden/make_full_batch_golden.py): the loss and, per parameter, a sample of gradient rows.

Products and per-element operations are bit-exact; what differs from the reference's CPU evaluation is
the association of fp32 sums (split-K weight gradients over 12608 / 4096 tokens, row sums of
LayerNorm / softmax, bias gradients), hence tolerances relative to each gradient tensor's largest
magnitude, which the fixture records."""
import pathlib

import numpy as np
import pytest
import torch

from conftest import assert_close_nan
from full_batch_cases import CASES, sample

from pam_b200 import steps

pytestmark = pytest.mark.gpu
GOLDEN = pathlib.Path(__file__).parent / "golden" / "full_batch_golden.npz"


@pytest.mark.parametrize("name", ["deit", "transformer"])
def test_full_batch_step_against_reference_fixture(name):
    import pam_b200 as pam
    if not GOLDEN.exists():
        pytest.skip("fixture not generated")
    data = np.load(GOLDEN)
    if f"{name}/loss" not in data.files:
        pytest.skip(f"fixture holds no {name} step")
    dev = torch.device("cuda", 0)
    params, loss_of = CASES[name]()
    leaves = steps.to_device(params, dev)
    loss = loss_of(pam, leaves, lambda t: t.to(dev))
    loss.backward()
    want = torch.from_numpy(data[f"{name}/loss"])
    assert_close_nan(loss.detach().reshape(1), want, 2e-5, 0.0, "loss")
    worst, failures = 0.0, []
    for k, leaf in leaves.items():
        ref = torch.from_numpy(data[f"{name}/grad/{k}"])
        scale = float(data[f"{name}/grad_max/{k}"][0])
        got = sample(leaf.grad).cpu()
        # The gradient of a key projection's bias is zero in exact arithmetic (a constant added to every key
        # shifts all scores of a row alike, and softmax does not see it): both sides hold the rounding residue
        # of sums over all tokens, two orders of magnitude below the other biases' gradients.
        tol = 2e-2 if k.endswith(".k.b") else 2e-3
        if scale > 0 and not k.endswith(".k.b"):
            worst = max(worst, float((got - ref).abs().max()) / scale)
        try:
            assert_close_nan(got, ref, tol, tol * scale + 1e-12, f"grad {k}")
        except AssertionError as err:
            failures.append(str(err))
    print(f"{name}: largest sampled gradient deviation relative to the tensor's maximum: {worst:.2e}")
    assert not failures, "\n".join(failures)
