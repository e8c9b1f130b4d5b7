"""The plugin path on the GPU: modules built by the factories from configuration strings, after
``install_as_pam()``, exactly the way the reference's timm / fairseq forks build them.

A DeiT-tiny block is assembled as ``nn.Module``s from ``get_linear_factory`` / ``get_norm_factory``
/ ``get_conv_factory`` / ``get_function_dict`` (shared/modules/factories.py:103-121, 124-199,
220-298) with the configuration text the forks pass on their command lines
(timm/models/vision_transformer.py:55-98, 275-277, 306-328), given the same weights as the
functional graph of tests/test_gpu_block.py, and must reproduce it bit for bit: output, every
gradient, the parameters after one PAM Adam step; its ``state_dict`` keys must equal those of the
same block built from the stock torch modules (checkpoints interchange)."""
import pytest
import torch
from torch import nn

from conftest import assert_bits_equal
from test_gpu_block import BATCH, D, HEADS, MLP, TOKENS, KW, block, make_params

pytestmark = pytest.mark.gpu

LINEAR_CFG = '{"subtype": "pam", "dkwargs": {"approx_bwd": true}}'
FUNCTION_CFG = '{"type": "pam", "dkwargs": {"approx_bwd": true}}'
NORM_CFG = '{"subtype": "pam_ln", "dkwargs": {"approx_bwd": true}}'
CONV_CFG = '{"subtype": "pam", "dkwargs": {"approx_bwd": true}}'


class Attention(nn.Module):
    """The attention module of the timm fork, with the scale and softmax taken from the operator
    dictionary as well (what the configuration "PAM linear / LN / functional" adds)."""

    def __init__(self, dim, heads, linear_factory, ops):
        super().__init__()
        self.heads, self.scale, self.ops = heads, (dim // heads) ** -0.5, ops
        self.qkv = linear_factory(dim, dim * 3, bias=True)
        self.proj = linear_factory(dim, dim)

    def forward(self, x):
        B, N, C = x.shape
        qkv = self.qkv(x).reshape(B, N, 3, self.heads, C // self.heads).permute(2, 0, 3, 1, 4)
        q, k, v = qkv.unbind(0)
        attn = self.ops["bmm"](q.flatten(0, 1), k.transpose(-2, -1).flatten(0, 1))
        attn = self.ops["mul"](attn, self.scale)
        attn = self.ops["softmax"](attn, dim=-1)
        x = self.ops["bmm"](attn, v.flatten(0, 1)).view(B, self.heads, N, C // self.heads)
        return self.proj(x.transpose(1, 2).reshape(B, N, C))


class Mlp(nn.Module):
    def __init__(self, dim, hidden, linear_factory):
        super().__init__()
        self.fc1 = linear_factory(dim, hidden, bias=True)
        self.act = nn.GELU()
        self.fc2 = linear_factory(hidden, dim, bias=True)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


class Block(nn.Module):
    def __init__(self, dim, heads, hidden, norm_layer, linear_factory, ops):
        super().__init__()
        self.norm1 = norm_layer(dim)
        self.attn = Attention(dim, heads, linear_factory, ops)
        self.norm2 = norm_layer(dim)
        self.mlp = Mlp(dim, hidden, linear_factory)

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


NAMES = {"ln1": "norm1", "qkv": "attn.qkv", "proj": "attn.proj", "ln2": "norm2", "fc1": "mlp.fc1", "fc2": "mlp.fc2"}


def load(module, params):
    state = {}
    for key, value in params.items():
        stem, kind = key.split(".")
        state[f"{NAMES[stem]}.{'weight' if kind == 'w' else 'bias'}"] = value
    module.load_state_dict(state)


@pytest.fixture(scope="module")
def factories():
    import pam_b200
    assert torch.cuda.is_available(), "gpu-marked tests need a CUDA device"
    pam_b200.install_as_pam()
    import pam                                              # the reference's import names now resolve to this package
    from shared.modules import factories as f
    assert pam is pam_b200 and f is pam_b200.factories
    return f


def test_block_built_by_the_factories_equals_the_functional_graph(factories):
    import pam_b200 as pam
    from pam_b200 import optim
    dev = torch.device("cuda", 0)
    linear_factory = factories.get_linear_factory(LINEAR_CFG)
    norm_factory = factories.get_norm_factory(NORM_CFG)
    ops = factories.get_function_dict(FUNCTION_CFG)
    model = Block(D, HEADS, MLP, lambda d: norm_factory(d, eps=1e-6), linear_factory, ops).to(dev)
    assert isinstance(model.attn.qkv, pam.Linear) and isinstance(model.norm1, pam.LayerNorm)
    assert model.attn.qkv.approx_bwd is True and "pam." in repr(model.attn.qkv)

    stock = Block(D, HEADS, MLP, lambda d: nn.LayerNorm(d, eps=1e-6), nn.Linear,
                  factories.get_function_dict("torch"))
    assert list(model.state_dict().keys()) == list(stock.state_dict().keys())
    assert [tuple(v.shape) for v in model.state_dict().values()] == [tuple(v.shape) for v in stock.state_dict().values()]

    g = torch.Generator().manual_seed(2024)
    params = make_params(g)
    x = torch.randn(BATCH, TOKENS, D, generator=g)
    gy = torch.randn(BATCH, TOKENS, D, generator=g) / (TOKENS * D)
    load(model, params)

    xm = x.to(dev).requires_grad_()
    ym = model(xm)
    ym.backward(gy.to(dev))

    leaves = {k: torch.nn.Parameter(v.to(dev)) for k, v in params.items()}
    xf = x.to(dev).requires_grad_()
    yf = block(pam, leaves, xf)
    yf.backward(gy.to(dev))

    assert_bits_equal(ym, yf, "block output")
    assert_bits_equal(xm.grad, xf.grad, "input gradient")
    named = dict(model.named_parameters())
    for key, leaf in leaves.items():
        stem, kind = key.split(".")
        assert_bits_equal(named[f"{NAMES[stem]}.{'weight' if kind == 'w' else 'bias'}"].grad, leaf.grad, f"gradient of {key}")

    hyper = dict(lr=5e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.05, opt_functional_cfg="pam")
    opt_m, opt_f = optim.Adam(model.parameters(), **hyper), optim.Adam(list(leaves.values()), **hyper)
    opt_m.step()
    opt_f.step()
    for key, leaf in leaves.items():
        stem, kind = key.split(".")
        assert_bits_equal(named[f"{NAMES[stem]}.{'weight' if kind == 'w' else 'bias'}"], leaf, f"{key} after one PAM Adam step")
    state = opt_m.state[model.attn.qkv.weight]
    assert set(state.keys()) == {"step", "exp_avg", "exp_avg_sq"}


def test_patch_embedding_conv_from_the_conv_factory(factories):
    """The ViT patch embedding as the fork builds it (timm/layers/patch_embed.py:36,47): a stride-16
    convolution from the conv factory, equal to the functional conv2d."""
    import pam_b200 as pam
    dev = torch.device("cuda", 0)
    conv_factory = factories.get_conv_factory(CONV_CFG)
    conv = conv_factory(3, D, kernel_size=16, stride=16).to(dev)
    assert isinstance(conv, pam.Conv2d) and conv.approx_bwd is True
    stock = nn.Conv2d(3, D, kernel_size=16, stride=16)
    assert list(conv.state_dict().keys()) == list(stock.state_dict().keys())
    g = torch.Generator().manual_seed(7)
    images = torch.randn(2, 3, 224, 224, generator=g).to(dev).requires_grad_()
    out = conv(images)
    out.sum().backward()
    w = conv.weight.detach().clone().requires_grad_()
    b = conv.bias.detach().clone().requires_grad_()
    images2 = images.detach().clone().requires_grad_()
    want = pam.conv2d(images2, w, b, stride=16, **KW)
    want.sum().backward()
    assert_bits_equal(out, want, "patch embedding")
    assert_bits_equal(conv.weight.grad, w.grad, "patch embedding weight gradient")
    assert_bits_equal(images.grad, images2.grad, "patch embedding input gradient")


def test_function_dictionaries_on_cuda(factories):
    """Every named operator dictionary resolves and runs on CUDA tensors; the PAM entries are this
    package's kernels (factories.py:220-298)."""
    dev = torch.device("cuda", 0)
    a = torch.randn(4, 5, 6, device=dev)
    b = torch.randn(4, 6, 7, device=dev)
    for name in ("standard", "torch", "standard2", "pam", "pam_bmm_only", "pam_softmax_only"):
        ops = factories.get_function_dict(name)
        assert set(ops) >= {"mean", "mul", "div", "softmax", "bmm", "logsumexp", "log_softmax", "pow"}
        assert ops["bmm"](a, b).shape == (4, 5, 7)
        assert torch.isfinite(ops["softmax"](a, dim=-1)).all()
    import pam_b200 as pam
    pam_ops = factories.get_function_dict(FUNCTION_CFG)
    assert_bits_equal(pam_ops["bmm"](a, b), pam.bmm(a, b, approx_bwd=True), "dictionary bmm")
    assert_bits_equal(pam_ops["softmax"](a, dim=-1, dtype=torch.float32), pam.softmax(a, dim=-1, approx_bwd=True),
                      "dictionary softmax (unknown keyword arguments are dropped)")


@pytest.mark.parametrize("name", ["deit", "transformer"])
def test_full_models_built_by_the_factories_equal_the_functional_graphs(factories, name):
    """DeiT-tiny (12 blocks, d 192, 197 tokens) and the 6+6 transformer (d 512, vocabulary 10000) as
    modules built from the forks' configuration strings (pam_b200/models.py) against the functional
    graphs of pam_b200/steps.py — the form the oracle comparisons of test_gpu_steps.py use — with the
    same weights and batch: loss and every gradient bit for bit."""
    import pam_b200 as pam
    from pam_b200 import models, steps
    dev = torch.device("cuda", 0)
    cfgs = models.pam_cfgs(approx_bwd=True)
    g = torch.Generator().manual_seed(77)
    if name == "deit":
        cfg = steps.DeitConfig()
        params = steps.deit_params(cfg, g)
        images = torch.randn(2, cfg.channels, cfg.image, cfg.image, generator=g).to(dev)
        labels = torch.randint(0, cfg.classes, (2,), generator=g).to(dev)
        model = models.VisionTransformer(cfg, linear_cfg=cfgs["linear"], conv_cfg=cfgs["linear"], norm_cfg=cfgs["norm"],
                                         functional_cfg=cfgs["function"]).load_parameters(params).to(dev)
        got = torch.nn.functional.cross_entropy(model(images), labels)
        leaves = steps.to_device(params, dev)
        want = steps.deit_loss(pam, leaves, images, labels, cfg, KW)
        flat_of = {"patch_embed.proj.weight": "patch.w", "patch_embed.proj.bias": "patch.b", "cls_token": "cls", "pos_embed": "pos",
                   "norm.weight": "norm.w", "norm.bias": "norm.b", "head.weight": "head.w", "head.bias": "head.b"}
        stems = {"norm1": "ln1", "attn.qkv": "qkv", "attn.proj": "proj", "norm2": "ln2", "mlp.fc1": "fc1", "mlp.fc2": "fc2"}
        for i in range(cfg.depth):
            for dotted, stem in stems.items():
                flat_of[f"blocks.{i}.{dotted}.weight"] = f"blocks.{i}.{stem}.w"
                flat_of[f"blocks.{i}.{dotted}.bias"] = f"blocks.{i}.{stem}.b"
    else:
        cfg = steps.TransformerConfig()
        params = steps.transformer_params(cfg, g)
        src, prev_out, target = (t.to(dev) for t in steps.transformer_batch(cfg, g, sentences=2, length=32))
        model = models.Transformer(cfg, linear_cfg=cfgs["linear"], norm_cfg=cfgs["norm"], functional_cfg=cfgs["function"],
                                   loss_functional_cfg=cfgs["function"]).load_parameters(params).to(dev)
        got = model.loss(src, prev_out, target)
        leaves = steps.to_device(params, dev)
        want = steps.transformer_loss(pam, leaves, src, prev_out, target, cfg, KW)
        flat_of = {"encoder.embed_tokens.weight": "enc.embed", "decoder.embed_tokens.weight": "dec.embed"}
        attn = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "out_proj": "out"}
        for side, short, layers in (("encoder", "enc", cfg.encoder_layers), ("decoder", "dec", cfg.decoder_layers)):
            for i in range(layers):
                for kind, suffix in (("weight", "w"), ("bias", "b")):
                    for dotted, a in attn.items():
                        flat_of[f"{side}.layers.{i}.self_attn.{dotted}.{kind}"] = f"{short}.{i}.self.{a}.{suffix}"
                        if side == "decoder":
                            flat_of[f"{side}.layers.{i}.encoder_attn.{dotted}.{kind}"] = f"{short}.{i}.cross.{a}.{suffix}"
                    flat_of[f"{side}.layers.{i}.self_attn_layer_norm.{kind}"] = f"{short}.{i}.ln_self.{suffix}"
                    if side == "decoder":
                        flat_of[f"{side}.layers.{i}.encoder_attn_layer_norm.{kind}"] = f"{short}.{i}.ln_cross.{suffix}"
                    flat_of[f"{side}.layers.{i}.final_layer_norm.{kind}"] = f"{short}.{i}.ln_ffn.{suffix}"
                    flat_of[f"{side}.layers.{i}.fc1.{kind}"] = f"{short}.{i}.fc1.{suffix}"
                    flat_of[f"{side}.layers.{i}.fc2.{kind}"] = f"{short}.{i}.fc2.{suffix}"
    got.backward()
    want.backward()
    assert_bits_equal(got.detach().reshape(1), want.detach().reshape(1), "loss")
    named = dict(model.named_parameters())                   # (the tied output projection appears once)
    assert set(named) == set(flat_of), sorted(set(named) ^ set(flat_of))
    for dotted, flat in flat_of.items():
        got_grad = named[dotted].grad.reshape(leaves[flat].shape)
        if dotted == "patch_embed.proj.bias":
            # the convolution module adds its bias to the [batch, channels, h, w] output and autograd sums the
            # gradient over three dimensions; the functional graph's linear layer sums token rows with the
            # column-sum kernel: the same 392 terms in another order
            assert torch.allclose(got_grad, leaves[flat].grad, rtol=1e-5, atol=1e-7), "gradient of the patch bias"
        else:
            assert_bits_equal(got_grad, leaves[flat].grad, f"gradient of {dotted}")
