"""The PAM loss kernels against the sequences of operator calls they replace.

* `pam_opt.cross_entropy`'s gradient (pam/pam_opt.py:27-51) in one launch: every per-element step
  is the same scalar function as in the elementwise kernels and the softmax inside it is the fused
  softmax kernel's, so the result must equal the unfused chain bit for bit — with and without
  label smoothing, class weights, ignored rows and the mean reduction — and equal the oracle's
  composition to the tolerance of the softmax row sums.
* the label-smoothed loss from the logits (fairseq criterions/label_smoothed_cross_entropy.py:36-54
  over the PAM log-softmax): loss, nll and the gradient of the logits against the unfused chain of
  dictionary calls, within the association of the fp32 row sums (a 10000-class row is summed by
  eight warps in the kernel and by torch's blocked sum in the chain), tolerance stated per check.
"""
import pytest
import torch

from conftest import assert_bits_equal, assert_close_nan

pytestmark = pytest.mark.gpu

FUNCTION_CFG = '{"type": "pam", "dkwargs": {"approx_bwd": true}}'


@pytest.fixture(scope="module")
def env():
    import pam_b200
    from pam_b200 import factories, fused, pam_opt
    assert torch.cuda.is_available(), "gpu-marked tests need a CUDA device"
    return pam_b200, factories, fused, pam_opt, torch.device("cuda", 0)


def _unfused(fused_module):
    """Context in which pam_opt takes the chain of dictionary calls instead of the loss kernels
    (the softmax / logsumexp row kernels stay on)."""
    class Off:
        def __enter__(self):
            self.saved = fused_module.loss_supported
            fused_module.loss_supported = lambda *a, **k: False

        def __exit__(self, *exc):
            fused_module.loss_supported = self.saved
    return Off()


@pytest.mark.parametrize("classes", [10, 1000, 10000])
@pytest.mark.parametrize("smoothing,weighted,ignore,reduction", [
    (0.0, False, -100, "mean"), (0.1, False, -100, "mean"), (0.1, True, 3, "mean"), (0.0, True, -100, "sum"), (0.2, False, 0, "sum")])
def test_cross_entropy_gradient_equals_the_unfused_chain(env, oracle, classes, smoothing, weighted, ignore, reduction):
    pam, factories, fused, pam_opt, dev = env
    rows = 64 if classes < 10000 else 24
    g = torch.Generator().manual_seed(classes + int(100 * smoothing))
    x = (torch.randn(rows, classes, generator=g) * 3).to(dev)
    y = torch.randint(0, classes, (rows,), generator=g).to(dev)
    if ignore >= 0:                                       # (-100: torch's "nothing ignored" default; None is rejected by torch)
        y[::5] = ignore
    w = (torch.rand(classes, generator=g) + 0.5).to(dev) if weighted else None
    for cfg in ("pam", FUNCTION_CFG):
        ops = factories.get_function_dict(cfg)
        results = []
        for use_kernel in (True, False):
            xi = x.clone().requires_grad_()
            with (_unfused(fused) if not use_kernel else torch.enable_grad()):
                loss = pam_opt.cross_entropy(xi, y, w, ignore, reduction, smoothing, op_dict=ops)
                (loss * 1.7).backward()
            results.append(xi.grad)
        assert_bits_equal(results[0], results[1], f"cross-entropy gradient, {classes} classes, cfg {cfg}")
    # and against the oracle's composition on the CPU (softmax row sums associate differently)
    xc = x.cpu().clone().requires_grad_()
    oracle_ops = {k: getattr(oracle, k) for k in ("mul", "div", "softmax")}      # the chain of pam_opt over the CPU oracle's operators
    want = pam_opt.cross_entropy(xc, y.cpu(), None if w is None else w.cpu(), ignore, reduction, smoothing, op_dict=oracle_ops)
    (want * 1.7).backward()
    assert_close_nan(results[0], xc.grad, 1e-4, 1e-4 * float(xc.grad.abs().max()), "against the oracle")


@pytest.mark.parametrize("rows,classes,ignore", [(96, 10000, None), (512, 1000, 1), (33, 17, None), (4096, 10000, None)])
def test_label_smoothed_loss_from_logits(env, rows, classes, ignore):
    pam, factories, fused, pam_opt, dev = env
    ops = factories.get_function_dict(FUNCTION_CFG)
    g = torch.Generator().manual_seed(rows)
    x = (torch.randn(rows, classes, generator=g) * 2).to(dev)
    y = torch.randint(2, classes, (rows,), generator=g).to(dev)
    if ignore is not None:
        y[::7] = ignore
    out = []
    for use_kernel in (True, False):
        xi = x.clone().requires_grad_()
        with (_unfused(fused) if not use_kernel else torch.enable_grad()):
            loss, nll = pam_opt.label_smoothed_nll_loss(xi, y, 0.1, ignore, op_dict=ops)
            loss.backward()
        out.append((loss.detach(), nll.detach(), xi.grad))
    (loss_k, nll_k, dx_k), (loss_c, nll_c, dx_c) = out
    # sums of `rows` (nll) and rows x classes (smooth) fp32 terms in two different orders
    assert_close_nan(loss_k.reshape(1), loss_c.reshape(1), 2e-6, 0.0, "loss")
    assert_close_nan(nll_k.reshape(1), nll_c.reshape(1), 2e-6, 0.0, "nll")
    # the gradient's row constant is a sum of `classes` equal terms: relative 1e-5 of the largest entry
    assert_close_nan(dx_k, dx_c, 1e-5, 1e-5 * float(dx_c.abs().max()), "gradient of the logits")
    if ignore is not None:
        assert bool((dx_k[::7] == 0).all()), "ignored rows get no gradient"
