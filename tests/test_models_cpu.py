"""The module forms of the two models (pam_b200/models.py: layers created from configuration strings
through the factories, as the reference's forks create them) against the functional graphs of
pam_b200/steps.py at toy sizes on the CPU, over the oracle-backed fake library: loss and every
gradient bit for bit, and parameter names equal to those of the same model built from stock layers."""
import pytest
import torch

import cpu_backend
from conftest import assert_bits_equal

from test_steps_cpu import DEIT, KW, TRANSFORMER, workload


def _named_grads(model):
    return {k: v.grad for k, v in model.named_parameters()}


@pytest.mark.parametrize("name", ["deit", "transformer"])
def test_module_form_equals_functional_graph(oracle, monkeypatch, name):
    cpu_backend.install(monkeypatch)
    import pam_b200 as pam
    from pam_b200 import models
    cfgs = models.pam_cfgs(approx_bwd=True)
    params, loss_fn = workload(name)
    leaves = {k: v.clone().requires_grad_() for k, v in params.items()}
    want = loss_fn(pam, leaves)
    want.backward()

    if name == "deit":
        from pam_b200 import steps
        model = models.VisionTransformer(DEIT, linear_cfg=cfgs["linear"], conv_cfg=cfgs["linear"], norm_cfg=cfgs["norm"],
                                         functional_cfg=cfgs["function"]).load_parameters(params)
        g = torch.Generator().manual_seed(4)
        steps.deit_params(DEIT, g)                               # advance the generator past the parameters, as workload() does
        images = torch.randn(3, DEIT.channels, DEIT.image, DEIT.image, generator=g)
        labels = torch.randint(0, DEIT.classes, (3,), generator=g)
        got = torch.nn.functional.cross_entropy(model(images), labels)
        stock = models.VisionTransformer(DEIT)
        pairs = {"patch.w": "patch_embed.proj.weight", "cls": "cls_token", "pos": "pos_embed", "head.w": "head.weight",
                 "blocks.1.qkv.w": "blocks.1.attn.qkv.weight", "blocks.0.ln2.b": "blocks.0.norm2.bias",
                 "blocks.1.fc2.b": "blocks.1.mlp.fc2.bias", "norm.w": "norm.weight"}
    else:
        from pam_b200 import steps
        g = torch.Generator().manual_seed(3)
        steps.transformer_params(TRANSFORMER, g)                 # advance the generator past the parameters
        src, prev_out, target = steps.transformer_batch(TRANSFORMER, g, sentences=3, length=6)
        model = models.Transformer(TRANSFORMER, linear_cfg=cfgs["linear"], norm_cfg=cfgs["norm"],
                                   functional_cfg=cfgs["function"], loss_functional_cfg=cfgs["function"]).load_parameters(params)
        got = model.loss(src, prev_out, target)
        stock = models.Transformer(TRANSFORMER)
        pairs = {"enc.embed": "encoder.embed_tokens.weight", "dec.embed": "decoder.embed_tokens.weight",
                 "enc.1.self.q.w": "encoder.layers.1.self_attn.q_proj.weight", "dec.0.cross.out.b": "decoder.layers.0.encoder_attn.out_proj.bias",
                 "dec.1.ln_cross.w": "decoder.layers.1.encoder_attn_layer_norm.weight", "enc.0.fc1.w": "encoder.layers.0.fc1.weight",
                 "dec.1.ln_ffn.b": "decoder.layers.1.final_layer_norm.bias"}
    got.backward()
    assert_bits_equal(got.detach().reshape(1), want.detach().reshape(1), "loss")
    grads = _named_grads(model)
    for flat, dotted in pairs.items():
        assert_bits_equal(grads[dotted].reshape(leaves[flat].shape), leaves[flat].grad, f"gradient of {flat}")
    assert list(model.state_dict().keys()) == list(stock.state_dict().keys())
    assert isinstance(dict(model.named_modules())["blocks.0.attn.qkv" if name == "deit" else "encoder.layers.0.fc1"], pam.Linear)
