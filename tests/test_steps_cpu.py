"""The two training-step workloads (pam_b200/steps.py) at toy sizes on the CPU: the oracle's
restatement of the reference op library, and this package's host layer over the oracle-backed fake
library, against a fixture produced by the reference's own op library
(tests/golden/make_step_golden.py).  Every value is compared bit for bit: on the CPU all three run
the same operations with the same torch.sum reductions."""
import pathlib

import numpy as np
import pytest
import torch

import cpu_backend
from conftest import assert_bits_equal

from pam_b200 import steps

KW = dict(approx_bwd=True)
LR, BETAS, EPS, WD = 5e-4, (0.9, 0.98), 1e-8, 0.05
DEIT = steps.DeitConfig(image=16, patch=8, dim=24, depth=2, heads=3, mlp=48, classes=10)
TRANSFORMER = steps.TransformerConfig(vocab=40, dim=16, ffn=32, heads=4, encoder_layers=2, decoder_layers=2)


@pytest.fixture(scope="module")
def step_golden():
    data = np.load(pathlib.Path(__file__).parent / "golden" / "step_golden.npz")
    return {k: torch.from_numpy(data[k]) for k in data.files}


def workload(name, dev="cpu"):
    """(parameters, loss function of (ops, parameters)) exactly as the fixture's generator built
    them; the batch tensors are placed on `dev`, the parameters stay on the CPU."""
    if name == "deit":
        g = torch.Generator().manual_seed(4)
        params = steps.deit_params(DEIT, g)
        images = torch.randn(3, DEIT.channels, DEIT.image, DEIT.image, generator=g)
        labels = torch.randint(0, DEIT.classes, (3,), generator=g).to(dev)
        images = images.to(dev)
        return params, lambda ops, p: steps.deit_loss(ops, p, images, labels, DEIT, KW)
    g = torch.Generator().manual_seed(3)
    params = steps.transformer_params(TRANSFORMER, g)
    src, prev_out, target = (t.to(dev) for t in steps.transformer_batch(TRANSFORMER, g, sentences=3, length=6))
    return params, lambda ops, p: steps.transformer_loss(ops, p, src, prev_out, target, TRANSFORMER, KW)


def check_step(name, golden, ops, update):
    params, loss_fn = workload(name)
    leaves = {k: v.clone().requires_grad_() for k, v in params.items()}
    loss = loss_fn(ops, leaves)
    loss.backward()
    assert_bits_equal(loss.detach().reshape(1), golden[f"{name}/loss"], "loss")
    for k, leaf in leaves.items():
        assert_bits_equal(leaf.grad, golden[f"{name}/grad/{k}"], f"grad {k}")
    updated = update(leaves)
    for k in leaves:
        assert_bits_equal(updated[k], golden[f"{name}/updated/{k}"], f"updated {k}")
    with torch.no_grad():
        after = loss_fn(ops, {k: v.detach() for k, v in updated.items()})
    assert_bits_equal(after.reshape(1), golden[f"{name}/loss_after"], "loss after the update")


@pytest.mark.parametrize("name", ["deit", "transformer"])
def test_oracle_step_equals_reference(step_golden, oracle, name):
    def update(leaves):
        return {k: oracle.adam_step(v.detach(), v.grad, torch.zeros_like(v), torch.zeros_like(v), step=1, lr=LR,
                                    betas=BETAS, eps=EPS, weight_decay=WD)[0] for k, v in leaves.items()}
    check_step(name, step_golden, oracle, update)


@pytest.mark.parametrize("name", ["deit", "transformer"])
def test_host_layer_step_equals_reference(step_golden, oracle, monkeypatch, name):
    cpu_backend.install(monkeypatch)
    import pam_b200 as pam
    from pam_b200 import optim

    def update(leaves):
        opt = optim.Adam(list(leaves.values()), lr=LR, betas=BETAS, eps=EPS, weight_decay=WD, opt_functional_cfg="pam")
        opt.step()
        return leaves
    check_step(name, step_golden, pam, update)
