"""The two models of the reference's experiments as ``nn.Module``s built through the plugin API.

These are the module graphs of the reference's forks, reduced to what the PAM path touches, with
every swappable layer created the way the forks create it — from configuration strings through
``get_linear_factory / get_conv_factory / get_norm_factory / get_function_dict``
(shared/modules/factories.py:103-121, 124-199, 220-298):

* ``VisionTransformer``: DeiT-tiny of the timm fork (timm/models/vision_transformer.py:55-98,
  275-328, 437-440; timm/layers/mlp.py:25-38; timm/layers/patch_embed.py:36-47): patch embedding
  from the conv factory, qkv / proj / fc1 / fc2 / head from the linear factory, both attention
  products through the operator dictionary's ``bmm``.  On top of the fork's hooks the norm layers
  come from the norm factory and the attention scale and softmax from the operator dictionary
  (the configuration "PAM linear / LN / functional").
* ``Transformer``: the encoder-decoder of the fairseq fork at ``transformer_iwslt_de_en`` sizes
  (fairseq/modules/transformer_layer.py:38-84, 270-360; multihead_attention.py:96-149, 618-783;
  models/transformer/transformer_decoder.py:149-173, 455-463): projections and feed-forward layers
  from the linear factory, LayerNorms from the norm factory, query scaling, attention products,
  softmax and the embedding scale through the operator dictionary, decoder input and output
  embeddings tied so that the vocabulary projection is a layer of the linear factory too, and the
  label-smoothed loss of criterions/label_smoothed_cross_entropy.py:36-54 through the loss
  operator dictionary.

Parameter names follow the forks (``blocks.3.attn.qkv.weight``, ``encoder.layers.0.self_attn.
q_proj.weight`` ...), so state dictionaries interchange with models built from the stock layers.
``load_parameters`` fills a model from the flat dictionaries of ``pam_b200.steps`` (the functional
form of the same graphs), which is how the tests check that both forms agree bit for bit.
"""
import math

import torch
import torch.nn.functional as F
from torch import nn

from . import factories, fused
from .pam_opt import _pam_binding
from .steps import DeitConfig, TransformerConfig, sinusoidal_positions


# ---- DeiT-tiny (timm fork) -----------------------------------------------------------------------------

class Attention(nn.Module):
    def __init__(self, dim, num_heads, qkv_bias, linear_factory, ops):
        super().__init__()
        self.num_heads, self.scale, self.ops = num_heads, (dim // num_heads) ** -0.5, ops
        self.qkv = linear_factory(dim, dim * 3, bias=qkv_bias)
        self.proj = linear_factory(dim, dim)

    def forward(self, x):
        B, N, C = x.shape
        qkv = self.qkv(x)
        bound = _pam_binding(self.ops, ("bmm", "softmax", "mul"))
        if bound is not None and fused.attention_supported(qkv, self.num_heads, bound.get("approx_bwd", False)):
            # the same products, scaling and softmax on strided views of qkv: no copies around them
            return self.proj(fused.attention_qkv(qkv, self.num_heads, self.scale, offset=bound.get("offset")))
        qkv = qkv.reshape(B, N, 3, self.num_heads, C // self.num_heads).permute(2, 0, 3, 1, 4)
        q, k, v = qkv.unbind(0)
        attn = self.ops["bmm"](q.flatten(0, 1), k.transpose(-2, -1).flatten(0, 1))
        attn = self.ops["softmax"](self.ops["mul"](attn, self.scale), dim=-1)
        x = self.ops["bmm"](attn, v.flatten(0, 1)).view(B, self.num_heads, N, C // self.num_heads)
        return self.proj(x.transpose(1, 2).reshape(B, N, C))


class Mlp(nn.Module):
    def __init__(self, in_features, hidden_features, linear_factory):
        super().__init__()
        self.fc1 = linear_factory(in_features, hidden_features, bias=True)
        self.act = nn.GELU()
        self.fc2 = linear_factory(hidden_features, in_features, bias=True)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


class Block(nn.Module):
    def __init__(self, dim, num_heads, hidden, norm_layer, linear_factory, ops):
        super().__init__()
        self.norm1 = norm_layer(dim)
        self.attn = Attention(dim, num_heads, True, linear_factory, ops)
        self.norm2 = norm_layer(dim)
        self.mlp = Mlp(dim, hidden, linear_factory)

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


class PatchEmbed(nn.Module):
    def __init__(self, patch, channels, dim, conv_factory):
        super().__init__()
        self.proj = conv_factory(channels, dim, kernel_size=patch, stride=patch)

    def forward(self, x):
        return self.proj(x).flatten(2).transpose(1, 2)


class VisionTransformer(nn.Module):
    def __init__(self, cfg=DeitConfig(), linear_cfg="standard", conv_cfg="standard", norm_cfg="layer_norm",
                 functional_cfg="torch"):
        super().__init__()
        self.cfg = cfg
        linear_factory = factories.get_linear_factory(linear_cfg)
        norm_factory = factories.get_norm_factory(norm_cfg)
        norm_layer = lambda dim: norm_factory(dim, eps=cfg.eps)
        ops = factories.get_function_dict(functional_cfg)
        self.patch_embed = PatchEmbed(cfg.patch, cfg.channels, cfg.dim, factories.get_conv_factory(conv_cfg))
        self.cls_token = nn.Parameter(torch.zeros(1, 1, cfg.dim))
        self.pos_embed = nn.Parameter(torch.zeros(1, cfg.tokens, cfg.dim))
        self.blocks = nn.Sequential(*[Block(cfg.dim, cfg.heads, cfg.mlp, norm_layer, linear_factory, ops)
                                      for _ in range(cfg.depth)])
        self.norm = norm_layer(cfg.dim)
        self.head = linear_factory(cfg.dim, cfg.classes)

    def forward(self, images):
        x = self.patch_embed(images)
        x = torch.cat([self.cls_token.expand(x.shape[0], -1, -1), x], dim=1) + self.pos_embed
        x = self.norm(self.blocks(x))
        return self.head(x[:, 0])

    def load_parameters(self, p):
        """Fills the model from the flat dictionary of `steps.deit_params`."""
        names = {"ln1": "norm1", "qkv": "attn.qkv", "proj": "attn.proj", "ln2": "norm2", "fc1": "mlp.fc1", "fc2": "mlp.fc2"}
        state = {"patch_embed.proj.weight": p["patch.w"], "patch_embed.proj.bias": p["patch.b"], "cls_token": p["cls"],
                 "pos_embed": p["pos"], "norm.weight": p["norm.w"], "norm.bias": p["norm.b"],
                 "head.weight": p["head.w"], "head.bias": p["head.b"]}
        for key, value in p.items():
            if key.startswith("blocks."):
                _, index, rest = key.split(".", 2)
                stem, kind = rest.split(".")
                state[f"blocks.{index}.{names[stem]}.{'weight' if kind == 'w' else 'bias'}"] = value
        self.load_state_dict({k: v.detach() for k, v in state.items()})
        return self


# ---- encoder-decoder transformer (fairseq fork) ----------------------------------------------------------

class MultiheadAttention(nn.Module):
    """The explicit (non-fused) branch the fork takes when custom operators are configured."""

    def __init__(self, embed_dim, num_heads, linear_factory, op_dict):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, embed_dim // num_heads
        self.scaling = self.head_dim ** -0.5
        self.k_proj = linear_factory(embed_dim, embed_dim, bias=True)
        self.v_proj = linear_factory(embed_dim, embed_dim, bias=True)
        self.q_proj = linear_factory(embed_dim, embed_dim, bias=True)
        self.out_proj = linear_factory(embed_dim, embed_dim, bias=True)
        self.gain_op, self.bmm_op, self.softmax_op = op_dict["mul"], op_dict["bmm"], op_dict["softmax"]
        self.ops = op_dict

    def forward(self, query, memory, attn_mask=None):
        B, T, d = query.shape
        S, H, hd = memory.shape[1], self.num_heads, self.head_dim
        q = self.gain_op(self.q_proj(query), self.scaling)
        k, v = self.k_proj(memory), self.v_proj(memory)
        bound = _pam_binding(self.ops, ("bmm", "softmax"))
        if bound is not None and fused.attention_heads_supported(q, k, v, H, attn_mask, bound.get("approx_bwd", False)):
            # the same products, mask and softmax on strided views of the projections: no copies around them
            return self.out_proj(fused.attention_heads(q, k, v, H, attn_mask, offset=bound.get("offset")))
        split = lambda t, L: t.reshape(B, L, H, hd).transpose(1, 2).reshape(B * H, L, hd)
        w = self.bmm_op(split(q, T), split(k, S).transpose(1, 2))
        if attn_mask is not None:
            w = w + attn_mask
        w = self.softmax_op(w, dim=-1)
        ctx = self.bmm_op(w, split(v, S)).reshape(B, H, T, hd).transpose(1, 2).reshape(B, T, d)
        return self.out_proj(ctx)


class TransformerLayer(nn.Module):
    """Post-norm encoder layer, or decoder layer when `cross` is set (transformer_layer.py)."""

    def __init__(self, cfg, cross, linear_factory, norm_layer, op_dict):
        super().__init__()
        self.self_attn = MultiheadAttention(cfg.dim, cfg.heads, linear_factory, op_dict)
        self.self_attn_layer_norm = norm_layer(cfg.dim)
        if cross:
            self.encoder_attn = MultiheadAttention(cfg.dim, cfg.heads, linear_factory, op_dict)
            self.encoder_attn_layer_norm = norm_layer(cfg.dim)
        self.fc1 = linear_factory(cfg.dim, cfg.ffn)
        self.fc2 = linear_factory(cfg.ffn, cfg.dim)
        self.final_layer_norm = norm_layer(cfg.dim)
        self.cross = cross

    def forward(self, x, memory=None, self_mask=None):
        x = self.self_attn_layer_norm(x + self.self_attn(x, x, self_mask))
        if self.cross:
            x = self.encoder_attn_layer_norm(x + self.encoder_attn(x, memory))
        return self.final_layer_norm(x + self.fc2(torch.relu(self.fc1(x))))


class _Stack(nn.Module):
    def __init__(self, cfg, layers, cross, linear_factory, norm_layer, op_dict):
        super().__init__()
        self.cfg, self.op_dict = cfg, op_dict
        self.embed_tokens = nn.Embedding(cfg.vocab, cfg.dim, padding_idx=cfg.pad)
        self.embed_scale = math.sqrt(cfg.dim)
        self.layers = nn.ModuleList([TransformerLayer(cfg, cross, linear_factory, norm_layer, op_dict) for _ in range(layers)])

    def embed(self, tokens):
        x = self.op_dict["mul"](self.embed_scale, self.embed_tokens(tokens))
        return x + sinusoidal_positions(tokens.shape[1], self.cfg.dim, self.cfg.pad, tokens.device)


class Transformer(nn.Module):
    def __init__(self, cfg=TransformerConfig(), linear_cfg="standard", norm_cfg="layer_norm", functional_cfg="torch",
                 loss_functional_cfg="torch"):
        super().__init__()
        self.cfg = cfg
        linear_factory = factories.get_linear_factory(linear_cfg)
        norm_factory = factories.get_norm_factory(norm_cfg)
        norm_layer = lambda dim: norm_factory(dim, eps=cfg.eps)
        op_dict = factories.get_function_dict(functional_cfg)
        self.loss_ops = factories.get_function_dict(loss_functional_cfg)
        self.encoder = _Stack(cfg, cfg.encoder_layers, False, linear_factory, norm_layer, op_dict)
        self.decoder = _Stack(cfg, cfg.decoder_layers, True, linear_factory, norm_layer, op_dict)
        # the decoder's input and output embeddings are shared: the output projection is a layer of the
        # linear factory whose weight is the embedding table (transformer_decoder.py:455-463)
        self.decoder.output_projection = linear_factory(cfg.dim, cfg.vocab, bias=False)
        self.decoder.output_projection.weight = self.decoder.embed_tokens.weight

    def forward(self, src, prev_out):
        x = self.encoder.embed(src)
        for layer in self.encoder.layers:
            x = layer(x)
        T = prev_out.shape[1]
        future = torch.full((T, T), float("-inf"), device=src.device).triu(1)
        y = self.decoder.embed(prev_out)
        for layer in self.decoder.layers:
            y = layer(y, x, future)
        return self.decoder.output_projection(y)

    def loss(self, src, prev_out, target, fused=False):
        """Label-smoothed negative log-likelihood summed over the target tokens.  `fused` takes the
        loss from the logits in one row kernel each way (pam_opt.label_smoothed_nll_loss): the same
        values up to the association of the row sums."""
        ops, cfg = self.loss_ops, self.cfg
        if fused:
            from . import pam_opt
            logits = self(src, prev_out).reshape(-1, cfg.vocab)
            return pam_opt.label_smoothed_nll_loss(logits, target.reshape(-1), cfg.label_smoothing, op_dict=ops)[0]
        lprobs = ops["log_softmax"](self(src, prev_out).reshape(-1, cfg.vocab), dim=-1)
        nll = -lprobs.gather(-1, target.reshape(-1, 1)).sum()
        smooth = -lprobs.sum()
        eps_i = ops["div"](cfg.label_smoothing, cfg.vocab - 1)
        return ops["mul"](nll, 1.0 - cfg.label_smoothing - eps_i) + ops["mul"](smooth, eps_i)

    def load_parameters(self, p):
        """Fills the model from the flat dictionary of `steps.transformer_params`."""
        attn = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "out": "out_proj"}
        state = {"encoder.embed_tokens.weight": p["enc.embed"], "decoder.embed_tokens.weight": p["dec.embed"],
                 "decoder.output_projection.weight": p["dec.embed"]}
        for key, value in p.items():
            parts = key.split(".")
            if parts[1] == "embed":
                continue
            side = "encoder" if parts[0] == "enc" else "decoder"
            base = f"{side}.layers.{parts[1]}."
            kind = "weight" if parts[-1] == "w" else "bias"
            if parts[2] in ("self", "cross"):
                module = "self_attn" if parts[2] == "self" else "encoder_attn"
                state[f"{base}{module}.{attn[parts[3]]}.{kind}"] = value
            else:
                module = {"ln_self": "self_attn_layer_norm", "ln_cross": "encoder_attn_layer_norm",
                          "ln_ffn": "final_layer_norm", "fc1": "fc1", "fc2": "fc2"}[parts[2]]
                state[f"{base}{module}.{kind}"] = value
        self.load_state_dict({k: v.detach() for k, v in state.items()})
        return self


PAM_LINEAR_CFG = '{"subtype": "pam", "dkwargs": {"approx_bwd": true}}'
PAM_NORM_CFG = '{"subtype": "pam_ln", "dkwargs": {"approx_bwd": true}}'
PAM_FUNCTION_CFG = '{"type": "pam", "dkwargs": {"approx_bwd": true}}'


def pam_cfgs(approx_bwd=True):
    """The configuration strings of an all-PAM run (the forks' --linear-cfg / --norm-cfg /
    --functional-cfg / --loss-functional-cfg values), with the gradient mode filled in."""
    flag = "true" if approx_bwd else "false"
    return dict(linear=PAM_LINEAR_CFG.replace("true", flag), norm=PAM_NORM_CFG.replace("true", flag),
                function=PAM_FUNCTION_CFG.replace("true", flag))
