"""The two training steps the reference's experiments run, as synthetic workloads written against
an operator namespace.

`ops` is any namespace with the reference's function front-ends (`linear bmm mul div softmax
log_softmax layer_norm`, pam/pam_ops.py) — this package on CUDA tensors, or a CPU restatement with
the same signatures — so one graph definition serves the product, the parity tests and the
benchmark.  `kw` carries the keyword-only settings (`offset`, `approx_bwd`) to every call, the way
the reference's factories bind them (shared/modules/factories.py:213-217).

* `deit_*`: DeiT-tiny of the timm fork (submodules/timm/timm/models/deit.py:195-201 and
  vision_transformer.py:55-98, 437-440): patch 16, 224x224x3 images, d = 192, 12 blocks, 3 heads,
  MLP 768.  qkv / proj / fc1 / fc2 / head and the patch embedding (a stride-16 convolution, i.e.
  unfold + matrix product, pam/pam_ops.py:118-158) are PAM products, both attention products go
  through `bmm`; on top of what the fork hooks, the LayerNorms, the attention scale and the softmax
  use PAM arithmetic as well.  GELU and the cross-entropy loss are ordinary, as in the fork.
* `transformer_*`: the 6+6-layer encoder-decoder of the fairseq fork at `transformer_iwslt_de_en`
  sizes (submodules/fairseq/fairseq/models/transformer/transformer_legacy.py:226-236): d = 512,
  FFN 1024, 4 heads, post-norm, ReLU, sinusoidal positions, embedding scale sqrt(d) through `mul`,
  decoder input and output embeddings shared so the vocabulary projection is a PAM product, query
  scaling through `mul` (fairseq/modules/multihead_attention.py:618), label-smoothed loss through
  `log_softmax`, `div` and `mul` (fairseq/criterions/label_smoothed_cross_entropy.py:36-54).

Parameters are plain dicts of fp32 tensors (created on the CPU from a generator; move them with
`to_device`).  Dropout is zero: the workloads are deterministic.
"""
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


# ---- DeiT-tiny -------------------------------------------------------------------------------------

@dataclass(frozen=True)
class DeitConfig:
    image: int = 224
    patch: int = 16
    channels: int = 3
    dim: int = 192
    depth: int = 12
    heads: int = 3
    mlp: int = 768
    classes: int = 10
    eps: float = 1e-6

    @property
    def tokens(self):
        return (self.image // self.patch) ** 2 + 1


def _trunc_normal(g, *shape, std=0.02):
    return torch.nn.init.trunc_normal_(torch.empty(*shape), std=std, generator=g)


def deit_params(cfg, g):
    """trunc_normal(0.02) weights, zero biases, unit LayerNorm gains (vision_transformer.py:358,
    376-383)."""
    d = cfg.dim
    p = {
        "patch.w": _trunc_normal(g, d, cfg.channels, cfg.patch, cfg.patch), "patch.b": torch.zeros(d),
        "cls": _trunc_normal(g, 1, 1, d), "pos": _trunc_normal(g, 1, cfg.tokens, d),
        "norm.w": torch.ones(d), "norm.b": torch.zeros(d),
        "head.w": _trunc_normal(g, cfg.classes, d), "head.b": torch.zeros(cfg.classes),
    }
    for i in range(cfg.depth):
        b = f"blocks.{i}."
        p.update({
            b + "ln1.w": torch.ones(d), b + "ln1.b": torch.zeros(d),
            b + "qkv.w": _trunc_normal(g, 3 * d, d), b + "qkv.b": torch.zeros(3 * d),
            b + "proj.w": _trunc_normal(g, d, d), b + "proj.b": torch.zeros(d),
            b + "ln2.w": torch.ones(d), b + "ln2.b": torch.zeros(d),
            b + "fc1.w": _trunc_normal(g, cfg.mlp, d), b + "fc1.b": torch.zeros(cfg.mlp),
            b + "fc2.w": _trunc_normal(g, d, cfg.mlp), b + "fc2.b": torch.zeros(d),
        })
    return p


def deit_forward(ops, p, images, cfg, kw):
    """Logits [batch, classes] of `images` [batch, channels, image, image]."""
    B, d, P = images.shape[0], cfg.dim, cfg.patch
    side = cfg.image // P
    # stride = kernel = patch: unfolding is a reshape; columns ordered (channel, row, column) like
    # F.unfold, which is the order of the flattened convolution weight
    patches = images.reshape(B, cfg.channels, side, P, side, P).permute(0, 2, 4, 1, 3, 5).reshape(B, side * side, -1)
    x = ops.linear(patches, p["patch.w"].reshape(d, -1), p["patch.b"], **kw)
    x = torch.cat([p["cls"].expand(B, -1, -1), x], dim=1) + p["pos"]
    hd = d // cfg.heads
    for i in range(cfg.depth):
        b = f"blocks.{i}."
        N = x.shape[1]
        h = ops.layer_norm(x, (d,), p[b + "ln1.w"], p[b + "ln1.b"], cfg.eps, **kw)
        qkv = ops.linear(h, p[b + "qkv.w"], p[b + "qkv.b"], **kw).reshape(B, N, 3, cfg.heads, hd).permute(2, 0, 3, 1, 4)
        q, k, v = (t.reshape(B * cfg.heads, N, hd) for t in qkv.unbind(0))
        attn = ops.bmm(q, k.transpose(-2, -1), **kw)
        attn = ops.softmax(ops.mul(attn, hd ** -0.5, **kw), dim=-1, **kw)
        ctx = ops.bmm(attn, v, **kw).reshape(B, cfg.heads, N, hd).transpose(1, 2).reshape(B, N, d)
        x = x + ops.linear(ctx, p[b + "proj.w"], p[b + "proj.b"], **kw)
        h = ops.layer_norm(x, (d,), p[b + "ln2.w"], p[b + "ln2.b"], cfg.eps, **kw)
        h = F.gelu(ops.linear(h, p[b + "fc1.w"], p[b + "fc1.b"], **kw))
        x = x + ops.linear(h, p[b + "fc2.w"], p[b + "fc2.b"], **kw)
    x = ops.layer_norm(x, (d,), p["norm.w"], p["norm.b"], cfg.eps, **kw)
    return ops.linear(x[:, 0], p["head.w"], p["head.b"], **kw)


def deit_loss(ops, p, images, labels, cfg, kw):
    return F.cross_entropy(deit_forward(ops, p, images, cfg, kw), labels)


def deit_macs(cfg, batch):
    """PAM multiply-accumulates of one forward pass (a training step runs three times as many:
    forward, input gradients, weight gradients)."""
    d, n = cfg.dim, cfg.tokens
    per_block = n * (d * 3 * d + d * d + 2 * d * cfg.mlp) + 2 * cfg.heads * n * n * (d // cfg.heads)
    return batch * ((n - 1) * cfg.channels * cfg.patch ** 2 * d + cfg.depth * per_block + d * cfg.classes)


# ---- 6+6 encoder-decoder transformer ------------------------------------------------------------------

@dataclass(frozen=True)
class TransformerConfig:
    vocab: int = 10000
    dim: int = 512
    ffn: int = 1024
    heads: int = 4
    encoder_layers: int = 6
    decoder_layers: int = 6
    pad: int = 1                 # fairseq/data/dictionary.py:24-27: bos 0, pad 1, eos 2, unk 3
    label_smoothing: float = 0.1
    eps: float = 1e-5


def _xavier(g, out_f, in_f, gain=1.0):
    bound = gain * math.sqrt(6.0 / (in_f + out_f))
    return (torch.rand(out_f, in_f, generator=g) * 2 - 1) * bound


def _attention_params(p, prefix, g, d):
    # q, k, v: xavier-uniform with gain 1/sqrt(2) (multihead_attention.py:182-196)
    for name, gain in (("q", 2 ** -0.5), ("k", 2 ** -0.5), ("v", 2 ** -0.5), ("out", 1.0)):
        p[prefix + name + ".w"] = _xavier(g, d, d, gain)
        p[prefix + name + ".b"] = torch.zeros(d)


def transformer_params(cfg, g):
    d = cfg.dim
    p = {}
    for side in ("enc", "dec"):
        emb = torch.randn(cfg.vocab, d, generator=g) * d ** -0.5     # transformer_base.py:194-198
        emb[cfg.pad] = 0
        p[side + ".embed"] = emb
    for side, layers in (("enc", cfg.encoder_layers), ("dec", cfg.decoder_layers)):
        for i in range(layers):
            b = f"{side}.{i}."
            _attention_params(p, b + "self.", g, d)
            p[b + "ln_self.w"], p[b + "ln_self.b"] = torch.ones(d), torch.zeros(d)
            if side == "dec":
                _attention_params(p, b + "cross.", g, d)
                p[b + "ln_cross.w"], p[b + "ln_cross.b"] = torch.ones(d), torch.zeros(d)
            p[b + "fc1.w"], p[b + "fc1.b"] = _xavier(g, cfg.ffn, d), torch.zeros(cfg.ffn)
            p[b + "fc2.w"], p[b + "fc2.b"] = _xavier(g, d, cfg.ffn), torch.zeros(d)
            p[b + "ln_ffn.w"], p[b + "ln_ffn.b"] = torch.ones(d), torch.zeros(d)
    return p


def sinusoidal_positions(length, dim, pad, device):
    """Rows pad+1 .. pad+length of fairseq's table (modules/sinusoidal_positional_embedding.py):
    [sin | cos] halves, frequencies 10000^(-i/(dim/2-1))."""
    half = dim // 2
    freq = torch.exp(torch.arange(half, dtype=torch.float32) * -(math.log(10000.0) / (half - 1)))
    pos = torch.arange(pad + 1, pad + 1 + length, dtype=torch.float32)[:, None] * freq[None, :]
    return torch.cat([torch.sin(pos), torch.cos(pos)], dim=1).to(device)


def _attention(ops, p, prefix, query, memory, heads, mask, kw):
    """fairseq MultiheadAttention's explicit branch: projections, PAM query scaling, bmm, additive
    mask, softmax, bmm, output projection.  Tensors are [batch, length, dim]."""
    B, T, d = query.shape
    S, hd = memory.shape[1], d // heads
    q = ops.mul(ops.linear(query, p[prefix + "q.w"], p[prefix + "q.b"], **kw), hd ** -0.5, **kw)
    k = ops.linear(memory, p[prefix + "k.w"], p[prefix + "k.b"], **kw)
    v = ops.linear(memory, p[prefix + "v.w"], p[prefix + "v.b"], **kw)
    split = lambda t, L: t.reshape(B, L, heads, hd).transpose(1, 2).reshape(B * heads, L, hd)
    w = ops.bmm(split(q, T), split(k, S).transpose(1, 2), **kw)
    if mask is not None:
        w = w + mask
    w = ops.softmax(w, dim=-1, **kw)
    ctx = ops.bmm(w, split(v, S), **kw).reshape(B, heads, T, hd).transpose(1, 2).reshape(B, T, d)
    return ops.linear(ctx, p[prefix + "out.w"], p[prefix + "out.b"], **kw)


def _embed(ops, table, tokens, cfg, kw):
    x = ops.mul(math.sqrt(cfg.dim), F.embedding(tokens, table, padding_idx=cfg.pad), **kw)
    return x + sinusoidal_positions(tokens.shape[1], cfg.dim, cfg.pad, tokens.device)


def transformer_forward(ops, p, src, prev_out, cfg, kw):
    """Decoder features projected onto the vocabulary: logits [batch, target length, vocab]."""
    d = cfg.dim
    ln = lambda x, name: ops.layer_norm(x, (d,), p[name + ".w"], p[name + ".b"], cfg.eps, **kw)

    def ffn(x, b):
        return ops.linear(torch.relu(ops.linear(x, p[b + "fc1.w"], p[b + "fc1.b"], **kw)), p[b + "fc2.w"], p[b + "fc2.b"], **kw)

    x = _embed(ops, p["enc.embed"], src, cfg, kw)
    for i in range(cfg.encoder_layers):
        b = f"enc.{i}."
        x = ln(x + _attention(ops, p, b + "self.", x, x, cfg.heads, None, kw), b + "ln_self")
        x = ln(x + ffn(x, b), b + "ln_ffn")
    memory = x
    T = prev_out.shape[1]
    future = torch.full((T, T), float("-inf"), device=src.device).triu(1)
    y = _embed(ops, p["dec.embed"], prev_out, cfg, kw)
    for i in range(cfg.decoder_layers):
        b = f"dec.{i}."
        y = ln(y + _attention(ops, p, b + "self.", y, y, cfg.heads, future, kw), b + "ln_self")
        y = ln(y + _attention(ops, p, b + "cross.", y, memory, cfg.heads, None, kw), b + "ln_cross")
        y = ln(y + ffn(y, b), b + "ln_ffn")
    return ops.linear(y, p["dec.embed"], **kw)


def transformer_loss(ops, p, src, prev_out, target, cfg, kw):
    """Label-smoothed negative log-likelihood summed over the target tokens
    (label_smoothed_cross_entropy.py:36-54 with reduce=True; no pad tokens in the synthetic batch)."""
    logits = transformer_forward(ops, p, src, prev_out, cfg, kw)
    lprobs = ops.log_softmax(logits.reshape(-1, cfg.vocab), dim=-1, **kw)
    nll = -lprobs.gather(-1, target.reshape(-1, 1)).sum()
    smooth = -lprobs.sum()
    eps_i = ops.div(cfg.label_smoothing, cfg.vocab - 1)           # scalar / scalar: a Python float
    return ops.mul(nll, 1.0 - cfg.label_smoothing - eps_i, **kw) + ops.mul(smooth, eps_i, **kw)


def transformer_batch(cfg, g, sentences=128, length=32):
    """Token ids uniform in [4, vocab): source, shifted decoder input (eos first, as fairseq's
    collater builds prev_output_tokens) and target."""
    src = torch.randint(4, cfg.vocab, (sentences, length), generator=g)
    target = torch.randint(4, cfg.vocab, (sentences, length), generator=g)
    prev_out = torch.cat([torch.full((sentences, 1), 2), target[:, :-1]], dim=1)
    return src, prev_out, target


def transformer_macs(cfg, sentences=128, length=32):
    """PAM multiply-accumulates of one forward pass."""
    d, t = cfg.dim, sentences * length
    attn = 4 * d * d * t + 2 * sentences * cfg.heads * length * length * (d // cfg.heads)
    ffn = 2 * d * cfg.ffn * t
    return cfg.encoder_layers * (attn + ffn) + cfg.decoder_layers * (2 * attn + ffn) + t * d * cfg.vocab


# ---- shared -------------------------------------------------------------------------------------------

def to_device(params, device, requires_grad=True):
    return {k: v.to(device).requires_grad_(requires_grad) for k, v in params.items()}
