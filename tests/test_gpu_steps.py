"""Full training steps (BASELINE configs 3 and 4) on the GPU through pam_b200.

* toy-size steps against the fixture produced by the reference's own op library
  (tests/golden/make_step_golden.py): loss, every gradient, every updated parameter and the loss
  after the update;
* the full-size models (DeiT-tiny: 12 blocks, d 192, 197 tokens; the 6+6 transformer: d 512, FFN
  1024, vocabulary 10000) with a small batch against the CPU oracle running the same graph.

Per-element operations and matrix products are bit-exact (see test_gpu_parity.py); what differs
between the GPU and the CPU here is the association of the fp32 row sums inside LayerNorm, softmax
and bias gradients, hence the relative tolerances, stated against the largest magnitude of each
tensor."""
import pathlib

import numpy as np
import pytest
import torch

from conftest import assert_close_nan

from pam_b200 import steps

pytestmark = pytest.mark.gpu

KW = dict(approx_bwd=True)
LR, BETAS, EPS, WD = 5e-4, (0.9, 0.98), 1e-8, 0.05


@pytest.fixture(scope="module")
def pam():
    import pam_b200
    assert torch.cuda.is_available(), "gpu-marked tests need a CUDA device"
    return pam_b200


@pytest.fixture(scope="module")
def step_golden():
    data = np.load(pathlib.Path(__file__).parent / "golden" / "step_golden.npz")
    return {k: torch.from_numpy(data[k]) for k in data.files}


def close(got, want, tol, what):
    scale = float(want.abs().max()) if want.numel() else 0.0
    assert_close_nan(got, want, tol, tol * scale + 1e-12, what)


@pytest.mark.parametrize("name", ["deit", "transformer"])
def test_toy_step_against_reference_fixture(pam, step_golden, name):
    from test_steps_cpu import workload
    from pam_b200 import optim
    dev = torch.device("cuda", 0)
    params, loss_fn = workload(name, dev)
    leaves = steps.to_device(params, dev)
    loss = loss_fn(pam, leaves)
    loss.backward()
    close(loss.detach().reshape(1), step_golden[f"{name}/loss"], 1e-5, "loss")
    for k, leaf in leaves.items():
        close(leaf.grad, step_golden[f"{name}/grad/{k}"], 2e-3, f"grad {k}")
    # the update from the fixture's gradients is a per-element rule: bit-exact
    for k, leaf in leaves.items():
        leaf.grad = step_golden[f"{name}/grad/{k}"].to(dev)
    optim.Adam(list(leaves.values()), lr=LR, betas=BETAS, eps=EPS, weight_decay=WD, opt_functional_cfg="pam").step()
    for k, leaf in leaves.items():
        want = step_golden[f"{name}/updated/{k}"]
        assert torch.equal(leaf.detach().cpu().view(torch.int32), want.view(torch.int32)), f"updated {k}"
    with torch.no_grad():
        after = loss_fn(pam, {k: v.detach() for k, v in leaves.items()})
    close(after.reshape(1), step_golden[f"{name}/loss_after"], 1e-5, "loss after the update")


def _compare_full(pam, oracle, params, loss_of, batch, tol_loss, tol_grad):
    dev = torch.device("cuda", 0)
    cpu = {k: v.clone().requires_grad_() for k, v in params.items()}
    lc = loss_of(oracle, cpu, *batch)
    lc.backward()
    gpu = steps.to_device(params, dev)
    lg = loss_of(pam, gpu, *(t.to(dev) for t in batch))
    lg.backward()
    close(lg.detach().reshape(1), lc.detach().reshape(1), tol_loss, "loss")
    worst = 0.0
    for k in params:
        ref = cpu[k].grad
        scale = float(ref.abs().max())
        if scale > 0:
            worst = max(worst, float((gpu[k].grad.cpu() - ref).abs().max()) / scale)
        close(gpu[k].grad, ref, tol_grad, f"grad {k}")
    return worst


def test_deit_tiny_full_model_step(pam, oracle):
    """BASELINE config 4's model at full size (batch 2): loss and all 152 gradients."""
    cfg = steps.DeitConfig()
    g = torch.Generator().manual_seed(44)
    params = steps.deit_params(cfg, g)
    images = torch.randn(2, cfg.channels, cfg.image, cfg.image, generator=g)
    labels = torch.randint(0, cfg.classes, (2,), generator=g)
    loss_of = lambda ops, p, x, y: steps.deit_loss(ops, p, x, y, cfg, KW)
    worst = _compare_full(pam, oracle, params, loss_of, (images, labels), 1e-4, 1e-3)
    print(f"largest gradient deviation relative to the tensor's maximum: {worst:.2e}")


def test_transformer_full_model_step(pam, oracle):
    """BASELINE config 3's model at full size (2 sentence pairs of 32 tokens): loss and gradients,
    through the shared-embedding vocabulary projection and the label-smoothed PAM loss."""
    cfg = steps.TransformerConfig()
    g = torch.Generator().manual_seed(33)
    params = steps.transformer_params(cfg, g)
    batch = steps.transformer_batch(cfg, g, sentences=2, length=32)
    loss_of = lambda ops, p, s, q, t: steps.transformer_loss(ops, p, s, q, t, cfg, KW)
    worst = _compare_full(pam, oracle, params, loss_of, batch, 1e-4, 1e-3)
    print(f"largest gradient deviation relative to the tensor's maximum: {worst:.2e}")
