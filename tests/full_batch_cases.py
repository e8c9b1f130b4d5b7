"""The two training workloads at the batch the benchmark runs them with, and the sampling of their
gradients that tests/golden/full_batch_golden.npz stores.  Shared by the fixture generator
(tests/golden/make_full_batch_golden.py, which runs them through the reference's operator library)
and by tests/test_gpu_full_batch.py; inputs and parameters are regenerated from the seeds."""
import torch

from pam_b200 import steps

KW = dict(approx_bwd=True)
ROWS, SAMPLE = 4, 64
DEIT_SEED, TRANSFORMER_SEED = 64, 4096


def sample_rows(shape):
    """Indices of the sampled rows of a parameter of this shape."""
    n = shape[0] if len(shape) > 1 else 1
    return sorted({(i * (n - 1)) // max(1, ROWS - 1) for i in range(min(ROWS, n))})


def sample(t):
    """Up to ROWS rows spread evenly over the first dimension, the first SAMPLE elements of each."""
    if t.dim() <= 1:
        return t.reshape(-1)[:SAMPLE].clone()
    flat = t.reshape(t.shape[0], -1)
    return torch.stack([flat[r, :SAMPLE] for r in sample_rows(t.shape)])


def deit_case():
    """DeiT-tiny (12 blocks, d 192, 197 tokens), 64 images of 3 x 224 x 224."""
    cfg = steps.DeitConfig()
    g = torch.Generator().manual_seed(DEIT_SEED)
    params = steps.deit_params(cfg, g)
    images = torch.randn(64, cfg.channels, cfg.image, cfg.image, generator=g)
    labels = torch.randint(0, cfg.classes, (64,), generator=g)
    return params, lambda ops, p, to=(lambda t: t): steps.deit_loss(ops, p, to(images), to(labels), cfg, KW)


def transformer_case():
    """6+6 encoder-decoder (d 512, FFN 1024, vocabulary 10000), 128 sentence pairs of 32 tokens."""
    cfg = steps.TransformerConfig()
    g = torch.Generator().manual_seed(TRANSFORMER_SEED)
    params = steps.transformer_params(cfg, g)
    batch = steps.transformer_batch(cfg, g)
    return params, lambda ops, p, to=(lambda t: t): steps.transformer_loss(ops, p, *(to(t) for t in batch), cfg, KW)


CASES = {"deit": deit_case, "transformer": transformer_case}
