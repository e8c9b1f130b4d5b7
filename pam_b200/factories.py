"""String / YAML configured factories — the plugin API of the reference's
``shared/modules/factories.py``, through which the timm and fairseq shims swap ``nn.Linear``,
``nn.LayerNorm``, ``torch.bmm``, ``softmax`` ... for their PAM versions.

Configuration grammar (unchanged):

* a module cfg is a known name (``"pam"``), or YAML/JSON text / a dict
  ``{"subtype": "pam", "dkwargs": {...}, "okwargs": {...}}`` — ``dkwargs`` are defaults that the
  call site may override, ``okwargs`` override the call site; keyword arguments the target does
  not accept are dropped with a warning; a list of such dicts (each with a ``type``) builds an
  ``nn.Sequential``;
* a function cfg is one of ``standard | torch | standard2 | pam | pam_bmm_only |
  pam_softmax_only`` or ``{"type": "pam", "dkwargs": {...}, "okwargs": {...}}`` and yields a dict
  with the keys ``mean mul div softmax bmm logsumexp log_softmax pow``.
"""
import copy
import inspect
import warnings

import torch
import yaml
from torch import nn
from torch.nn.modules.lazy import LazyModuleMixin
from torch.nn.parameter import Parameter, UninitializedParameter

import pam_b200 as pam


class CustomLinear(nn.Linear):
    """Placeholder subtype (``custom``) used to test that a factory is honoured."""


class CustomConv2d(nn.Conv2d):
    """Placeholder subtype (``custom``) used to test that a factory is honoured."""


class _PerChannel(nn.Module):
    """One learnable value per channel (dimension 1), combined with the input by ``_apply``."""
    _name = "value"
    _init = staticmethod(torch.nn.init.zeros_)

    def __init__(self, num_features=None):
        super().__init__()
        self.num_features = num_features
        setattr(self, self._name, Parameter(torch.empty(self.num_features)))
        self.reset_parameters()

    def _param(self):
        return getattr(self, self._name)

    def reset_parameters(self):
        self._init(self._param())

    def forward(self, x):
        shape = [dim if idx == 1 else 1 for idx, dim in enumerate(x.shape)]
        return self._apply_value(x, self._param().view(shape))

    def extra_repr(self):
        return f"{self.num_features}"


class Bias(_PerChannel):
    _name = "bias"
    _init = staticmethod(torch.nn.init.zeros_)

    @staticmethod
    def _apply_value(x, v):
        return x + v


class Gain(_PerChannel):
    _name = "gain"
    _init = staticmethod(torch.nn.init.ones_)

    @staticmethod
    def _apply_value(x, v):
        return x * v


class _LazyPerChannel(LazyModuleMixin):
    """Infers the channel count from the first input (factories.py:43-61, 83-100)."""

    def __init__(self):
        super().__init__(0)
        setattr(self, self._name, UninitializedParameter())

    def reset_parameters(self):
        if not self.has_uninitialized_params() and self.num_features != 0:
            super().reset_parameters()

    def initialize_parameters(self, input):
        if self.has_uninitialized_params():
            with torch.no_grad():
                self.num_features = input.shape[1]
                self._param().materialize((self.num_features,))
                self.reset_parameters()


class LazyBias(_LazyPerChannel, Bias):
    cls_to_become = Bias


class LazyGain(_LazyPerChannel, Gain):
    cls_to_become = Gain


def get_valid_kwargs(func, argdict):
    params = inspect.signature(func).parameters
    if any(p.kind == p.VAR_KEYWORD for p in params.values()):
        return argdict
    return {k: v for k, v in argdict.items() if k in params}


def call_valid_kwargs(func, kwargs_dict, args_tuple=tuple()):
    kwargs = get_valid_kwargs(func, kwargs_dict)
    if extra := sorted(set(kwargs_dict) - set(kwargs)):
        warnings.warn(f"Function {func} ignored extra arguments {extra}")
    return func(*args_tuple, **kwargs)


def get_module_factory(desc, factories):
    if isinstance(desc, str):
        if desc in factories:
            desc = {"subtype": desc}
        else:
            try:
                desc = yaml.safe_load(desc)
            except Exception:
                raise ValueError(f"Unknown linear function {desc}")
    if isinstance(desc, dict):
        target = factories[desc["subtype"].lower()]
        defaults, overrides = desc.get("dkwargs", {}), desc.get("okwargs", {})
        return lambda *a, **ka: call_valid_kwargs(target, {**defaults, **ka, **overrides}, a)
    if isinstance(desc, list):
        return get_sequential_factory(desc)
    raise ValueError(f"Unknown configuration {desc=}")


def get_linear_factory(desc):
    return get_module_factory(desc or "standard", {
        "standard": nn.Linear, "linear": nn.Linear, "pam": pam.Linear, "custom": CustomLinear})


def get_conv_factory(desc):
    return get_module_factory(desc or "standard", {
        "standard": nn.Conv2d, "conv2d": nn.Conv2d, "pam": pam.Conv2d, "custom": CustomConv2d})


def get_bias_factory(desc):
    return get_module_factory(desc or "standard", {"standard": Bias, "bias": Bias, "lazy_bias": LazyBias})


def get_gain_factory(desc):
    # the lazy variant is registered under "lazy_bias" in the reference as well (factories.py:164)
    return get_module_factory(desc or "standard", {"standard": Gain, "gain": Gain, "lazy_bias": LazyGain})


def get_activation_factory(desc):
    assert desc is not None, "Must specify activation type"
    return get_module_factory(desc, {"relu": nn.ReLU, "leaky_relu": nn.LeakyReLU})


def get_norm_factory(desc):
    assert desc is not None, "Must specify norm type"
    return get_module_factory(desc, {
        "batch_norm_2d": nn.BatchNorm2d, "bn2d": nn.BatchNorm2d,
        "layer_norm": nn.LayerNorm, "ln": nn.LayerNorm,
        "pam_layer_norm": pam.LayerNorm, "pam_ln": pam.LayerNorm})


_BY_TYPE = {
    "conv": get_conv_factory, "linear": get_linear_factory, "activation": get_activation_factory,
    "norm": get_norm_factory, "bias": get_bias_factory, "gain": get_gain_factory,
}


def get_sequential_factory(descriptions):
    parts = []
    for d in descriptions:
        if d["type"] not in _BY_TYPE:
            raise ValueError(f"Unknown factory type for {d}")
        parts.append(_BY_TYPE[d["type"]](d))
    return lambda **kwargs: torch.nn.Sequential(*[make(**kwargs) for make in parts])


_KEYS = ("mean", "mul", "div", "softmax", "bmm", "logsumexp", "log_softmax", "pow")


def _torch_dict():
    F = torch.nn.functional
    return dict(mean=torch.mean, mul=torch.mul, div=torch.div, softmax=F.softmax, bmm=torch.bmm,
                logsumexp=torch.logsumexp, log_softmax=F.log_softmax, pow=torch.pow)


def _pam_dict():
    return {k: getattr(pam, k) for k in _KEYS}


def get_function_dict(desc):
    """The eight-entry operator dictionary used by the attention, criterion and optimizer hooks."""
    if isinstance(desc, str):
        named = {
            "standard": _torch_dict, "torch": _torch_dict,
            "standard2": lambda: {**_torch_dict(), "softmax": pam.pam_experimental.torch_softmax2,
                                  "logsumexp": pam.pam_experimental.torch_logsumexp2,
                                  "log_softmax": pam.pam_experimental.torch_log_softmax2},
            "pam": _pam_dict,
            "pam_bmm_only": lambda: {**_torch_dict(), "bmm": pam.bmm},
            "pam_softmax_only": lambda: {**_torch_dict(), "softmax": pam.softmax},
        }
        if desc in named:
            return copy.copy(named[desc]())
        try:
            desc = yaml.safe_load(desc)
        except Exception:
            raise ValueError(f"Unknown function config {desc}")
    assert isinstance(desc, dict), f"Unknown function cfg {desc=}"
    assert desc["type"] in ("pam", "pam_bmm_only", "pam_softmax_only"), "Only support custom cfg for pam"
    defaults, overrides = desc.get("dkwargs", {}), desc.get("okwargs", {})
    # as in the reference (factories.py:291-298) the dict form wraps the full PAM dictionary
    # whatever `type` says
    def bind(func):
        def bound(*a, **ka):
            return call_valid_kwargs(func, {**defaults, **ka, **overrides}, a)
        # what the wrapper binds, for callers that can fuse a chain of these operators into one kernel
        bound.pam_function, bound.pam_kwargs = func, {**defaults, **overrides}
        return bound
    return {name: bind(func) for name, func in _pam_dict().items()}
