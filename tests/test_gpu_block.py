"""One DeiT-tiny transformer block and one optimizer step built from the PAM operators, on the GPU
through pam_b200 and on the CPU through the oracle's restatement of the reference op library.

The block follows the module graph of the reference's timm fork (qkv / proj / fc1 / fc2 through the
PAM linear factory, both attention products through the PAM bmm, timm/models/vision_transformer.py:
55-98) with the additions BASELINE config 4 names (PAM LayerNorm, PAM softmax and scale, PAM Adam
update rule).  Sizes are DeiT-tiny's (197 tokens, d = 192, 3 heads, MLP 768) with a small batch;
approx_bwd = True as in the configs.  Values that only differ by the association of fp32 sums
(row reductions, bias gradients) are compared with a relative tolerance."""

import pytest
import torch

from conftest import assert_close_nan

pytestmark = pytest.mark.gpu

D, HEADS, MLP, TOKENS, BATCH = 192, 3, 768, 197, 2
KW = dict(approx_bwd=True)


def make_params(g):
    def tn(*shape):
        return torch.nn.init.trunc_normal_(torch.empty(*shape), std=0.02, generator=g)
    return {
        "ln1.w": torch.ones(D), "ln1.b": torch.zeros(D), "qkv.w": tn(3 * D, D), "qkv.b": torch.zeros(3 * D),
        "proj.w": tn(D, D), "proj.b": torch.zeros(D), "ln2.w": torch.ones(D), "ln2.b": torch.zeros(D),
        "fc1.w": tn(MLP, D), "fc1.b": torch.zeros(MLP), "fc2.w": tn(D, MLP), "fc2.b": torch.zeros(D),
    }


def block(ops, p, x):
    B, N, C = x.shape
    h = ops.layer_norm(x, (C,), p["ln1.w"], p["ln1.b"], 1e-6, **KW)
    qkv = ops.linear(h, p["qkv.w"], p["qkv.b"], **KW).reshape(B, N, 3, HEADS, C // HEADS).permute(2, 0, 3, 1, 4)
    q, k, v = (t.reshape(B * HEADS, N, C // HEADS) for t in qkv.unbind(0))
    attn = ops.bmm(q, k.transpose(-2, -1), **KW)
    attn = ops.mul(attn, (C // HEADS) ** -0.5, **KW)
    attn = ops.softmax(attn, dim=-1, **KW)
    ctx = ops.bmm(attn, v, **KW).reshape(B, HEADS, N, C // HEADS).transpose(1, 2).reshape(B, N, C)
    x = x + ops.linear(ctx, p["proj.w"], p["proj.b"], **KW)
    h = ops.layer_norm(x, (C,), p["ln2.w"], p["ln2.b"], 1e-6, **KW)
    h = torch.nn.functional.gelu(ops.linear(h, p["fc1.w"], p["fc1.b"], **KW))
    return x + ops.linear(h, p["fc2.w"], p["fc2.b"], **KW)


def test_deit_block_forward_backward_and_adam_step(oracle):
    import pam_b200 as pam
    from pam_b200 import optim
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(2024)
    params = make_params(g)
    x = torch.randn(BATCH, TOKENS, D, generator=g)
    gy = torch.randn(BATCH, TOKENS, D, generator=g) / (TOKENS * D)

    cpu = {k: v.clone().requires_grad_() for k, v in params.items()}
    xc = x.clone().requires_grad_()
    yc = block(oracle, cpu, xc)
    yc.backward(gy)

    gpu = {k: torch.nn.Parameter(v.to(dev)) for k, v in params.items()}
    xg = x.to(dev).requires_grad_()
    yg = block(pam, gpu, xg)
    yg.backward(gy.to(dev))

    assert_close_nan(yg, yc, 2e-4, 2e-5, "block output")
    assert_close_nan(xg.grad, xc.grad, 5e-3, 5e-3 * float(xc.grad.abs().max()), "dx")
    for k in params:
        ref = cpu[k].grad
        assert_close_nan(gpu[k].grad, ref, 5e-3, 5e-3 * float(ref.abs().max()) + 1e-12, f"grad {k}")

    # one PAM Adam step from identical gradients must give identical parameters (per-element rule)
    opt = optim.Adam(list(gpu.values()), lr=5e-4, betas=(0.9, 0.98), eps=1e-8, weight_decay=0.05,
                     opt_functional_cfg="pam")
    for k in params:
        gpu[k].grad = cpu[k].grad.to(dev)
    opt.step()
    for k in params:
        want, _, _ = oracle.adam_step(params[k], cpu[k].grad, torch.zeros_like(params[k]), torch.zeros_like(params[k]),
                                      step=1, lr=5e-4, betas=(0.9, 0.98), eps=1e-8, weight_decay=0.05)
        assert torch.equal(gpu[k].detach().cpu().view(torch.int32), want.view(torch.int32)), f"adam {k}"


def test_vocabulary_loss_path(oracle):
    """The loss head of the 6+6-layer translation model of BASELINE config 3: tied output projection
    as a PAM GEMM onto a 10000-word vocabulary, PAM log-softmax over the vocabulary (rows of 10000:
    the CTA-per-row kernel), label-smoothed NLL with PAM scaling (fairseq criterions/
    label_smoothed_cross_entropy.py:36-54 through the operator dictionary), forward and backward."""
    import pam_b200 as pam
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(31)
    tokens, d_model, vocab, eps_ls = 96, 512, 10000, 0.1
    feats = torch.randn(tokens, d_model, generator=g)
    emb = torch.randn(vocab, d_model, generator=g) * d_model ** -0.5
    target = torch.randint(4, vocab, (tokens,), generator=g)

    def loss_fn(ops, feats, emb, target):
        logits = ops.linear(feats, emb, **KW)
        lprobs = ops.log_softmax(logits, dim=-1, **KW)
        nll = -lprobs.gather(-1, target.unsqueeze(-1)).sum()
        smooth = -lprobs.sum()
        eps_i = ops.div(eps_ls, vocab - 1)
        return ops.mul(nll, 1.0 - eps_ls - eps_i, **KW) + ops.mul(smooth, eps_i, **KW)

    fc, ec = feats.clone().requires_grad_(), emb.clone().requires_grad_()
    lc = loss_fn(oracle, fc, ec, target)
    lc.backward()
    fg, eg = feats.to(dev).requires_grad_(), emb.to(dev).requires_grad_()
    lg = loss_fn(pam, fg, eg, target.to(dev))
    lg.backward()
    assert_close_nan(lg.reshape(1), lc.reshape(1), 1e-4, 1e-4, "loss")
    assert_close_nan(fg.grad, fc.grad, 5e-3, 5e-3 * float(fc.grad.abs().max()), "d features")
    assert_close_nan(eg.grad, ec.grad, 5e-3, 5e-3 * float(ec.grad.abs().max()), "d embedding")
