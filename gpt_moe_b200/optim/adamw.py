"""AdamW with optional bf16 moments.

Same update rule and state keys (`step`, `exp_avg`, `exp_avg_sq`) as `torch.optim.AdamW`, which
the reference uses in fused mode (`model/gpt.py:284-293`), so optimizer state dicts interchange.
On CUDA all parameters of a group are updated by one multi-tensor kernel launch
(`csrc/fused/loss_optim.cu`) that also refreshes the bf16 compute copy of each weight; moments may be
bf16 while parameters stay fp32 (reference `runtime/precision.py:52-75`).
"""
from __future__ import annotations

import math
from typing import Iterable

import torch


class AdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2, moment_dtype: torch.dtype = torch.float32) -> None:
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, fused=True,
                        capturable=False, amsgrad=False, maximize=False, foreach=None, differentiable=False)
        super().__init__(params, defaults)
        self.moment_dtype = moment_dtype

    def state_dict(self):
        """torch layout; the device-side `step` tensors are synchronised with the host counters first."""
        for group in self.param_groups:
            for p in group["params"]:
                state = self.state.get(p)
                if state and "_host_step" in state:
                    state["step"].fill_(float(state["_host_step"]))
        sd = super().state_dict()
        for state in sd["state"].values():
            state.pop("_host_step", None)
        return sd

    def _init_state(self, p: torch.Tensor) -> dict:
        state = self.state[p]
        if not state:
            state["step"] = torch.zeros((), dtype=torch.float32, device=p.device)
            state["exp_avg"] = torch.zeros_like(p, dtype=self.moment_dtype)
            state["exp_avg_sq"] = torch.zeros_like(p, dtype=self.moment_dtype)
        return state

    @torch.no_grad()
    def step(self, closure=None):
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
            params = [p for p in group["params"] if p.grad is not None or getattr(p, "main_grad", None) is not None]
            if not params:
                continue
            states = [self._init_state(p) for p in params]
            if params[0].is_cuda:
                from ..ops import cuda_ops
                cuda_ops.adamw_step(params, states, lr, beta1, beta2, eps, wd)
                continue
            for p, state in zip(params, states):
                g = p.grad.float()
                state["step"] += 1
                t = float(state["step"])
                m, v = state["exp_avg"].float(), state["exp_avg_sq"].float()
                m.mul_(beta1).add_(g, alpha=1 - beta1)
                v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
                state["exp_avg"].copy_(m)
                state["exp_avg_sq"].copy_(v)
                p.mul_(1 - lr * wd)
                denom = (v.sqrt() / math.sqrt(1 - beta2 ** t)).add_(eps)
                p.addcdiv_(m, denom, value=-lr / (1 - beta1 ** t))


def configure_adamw_moments(optimizer: AdamW, use_bf16_adamw_moments: bool) -> None:
    """Set (or convert, keeping values and step counters) the moment dtype (reference `runtime/precision.py:52-75`)."""
    dtype = torch.bfloat16 if use_bf16_adamw_moments else torch.float32
    optimizer.moment_dtype = dtype
    for group in optimizer.param_groups:
        for p in group["params"]:
            state = optimizer.state[p]
            if state:
                state["exp_avg"] = state["exp_avg"].to(dtype)
                state["exp_avg_sq"] = state["exp_avg_sq"].to(dtype)
