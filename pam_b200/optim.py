"""PAM Adam — the optimizer of the reference's fairseq fork
(submodules/fairseq/fairseq/optim/adam.py:118-257) as a plain ``torch.optim.Optimizer``.

The update is AdamW-style (decoupled weight decay).  Every multiplication, division and square
root of the rule goes through the operator dictionary chosen by ``opt_functional_cfg``
(``"torch"``: ordinary arithmetic, ``"pam"``: PAM arithmetic); additions and subtractions are
ordinary fp32 operations.  State keys (``step``, ``exp_avg``, ``exp_avg_sq``) match the
reference's, so optimizer checkpoints interchange.

With the plain ``"pam"`` dictionary on CUDA tensors the whole per-tensor rule runs as one fused
kernel that rounds at the same points as the reference's chain of ~12 elementwise launches.
"""
import math

import torch

from . import factories, fused


class Adam(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, amsgrad=False,
                 opt_functional_cfg=None):
        if amsgrad:
            raise NotImplementedError("amsgrad is not supported by the PAM update rule")
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad)
        self.opt_functional_cfg = opt_functional_cfg
        self.op_dict = factories.get_function_dict(opt_functional_cfg or "torch")
        # the fused kernel implements the default PAM dictionary only (offset None)
        self._fusable = opt_functional_cfg == "pam"
        super().__init__(params, defaults)

    @property
    def supports_memory_efficient_fp16(self):
        return True

    @property
    def supports_flat_params(self):
        return True

    @staticmethod
    def _scalars(group, step):
        """step_size and decay, formed in double on the host (adam.py:240-243) and rounded to fp32
        only when they meet a tensor (pam/utils.py:13)."""
        beta1, beta2 = group["betas"]
        step_size = group["lr"] * math.sqrt(1 - beta2 ** step) / (1 - beta1 ** step)
        return step_size, group["weight_decay"] * group["lr"]

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        ops = self.op_dict
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            batches = {}             # step count -> tensors that share every scalar of the rule
            for p in group["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                if grad.is_sparse:
                    raise RuntimeError("Adam does not support sparse gradients, please consider SparseAdam instead")
                if grad.dtype in (torch.float16, torch.bfloat16):
                    grad = grad.float()
                half = p.dtype in (torch.float16, torch.bfloat16)
                p32 = p.float() if half else p

                state = self.state[p]
                if len(state) == 0:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros_like(p32)
                    state["exp_avg_sq"] = torch.zeros_like(p32)
                else:
                    state["exp_avg"] = state["exp_avg"].to(p32)
                    state["exp_avg_sq"] = state["exp_avg_sq"].to(p32)
                state["step"] += 1

                if self._fusable and not half and fused.adam_supported(p32, grad):
                    batches.setdefault(state["step"], []).append((p32, grad, state["exp_avg"], state["exp_avg_sq"]))
                    continue
                step_size, decay = self._scalars(group, state["step"])
                m, v = state["exp_avg"], state["exp_avg_sq"]
                m.copy_(ops["mul"](m, beta1) + ops["mul"](grad, 1 - beta1))
                v.copy_(ops["mul"](v, beta2))
                v += ops["mul"](ops["mul"](grad, grad), 1 - beta2)
                denom = ops["pow"](v, 0.5) + group["eps"]
                if group["weight_decay"] != 0:
                    p32 -= ops["mul"](p32, decay)
                p32 -= ops["mul"](ops["div"](m, denom), step_size)
                if half:
                    p.copy_(p32)
            for step, tensors in batches.items():
                step_size, decay = self._scalars(group, step)
                by_device = {}
                for t in tensors:
                    by_device.setdefault(t[0].device, []).append(t)
                for same_device in by_device.values():
                    fused.adam_step(same_device, beta1=beta1, beta2=beta2, eps=group["eps"],
                                    step_size=step_size, decay=decay if group["weight_decay"] != 0 else 0.0)
        return loss
