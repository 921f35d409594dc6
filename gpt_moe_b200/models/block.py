"""Pre-norm transformer block with weighted residual/main paths.

x = alpha_1 x + beta_1 Attn(norm(x));  x = alpha_2 x + beta_2 FFN(norm(x)) with learned scalars
alpha (`*_residual_scale`) and/or beta (`*_main_scale`), or a frozen (2L)^-0.5 `residual_scale`
when both are off (reference `model/block.py:19-134`).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn
from torch import Tensor

from ..ops import api
from .attention import AttentionContext, SelfAttention
from .mla import MLAttention
from .mlp import MLP
from .moe import MoE


def make_norm(gpt_config) -> nn.Module:
    return nn.RMSNorm(gpt_config.hidden_size) if gpt_config.norm_type.lower() == "rms" else nn.LayerNorm(gpt_config.hidden_size)


def norm_eps(norm: nn.Module, dtype: torch.dtype) -> float:
    return norm.eps if getattr(norm, "eps", None) is not None else torch.finfo(dtype).eps


def apply_norm(norm: nn.Module, x: Tensor) -> Tensor:
    if isinstance(norm, nn.RMSNorm):
        return api.rms_norm(x, norm.weight, norm_eps(norm, x.dtype))
    return norm(x)


class Block(nn.Module):
    def __init__(self, gpt_config, training_config, layer_idx: int = 0, ep_rank: int = 0, ep_size: int = 1) -> None:
        super().__init__()
        self.use_moe = gpt_config.use_moe
        self.use_weighted_residual_path = gpt_config.use_weighted_residual_path
        self.use_weighted_main_path = gpt_config.use_weighted_main_path
        if self.use_weighted_residual_path:
            self.attn_residual_scale = nn.Parameter(torch.full((1,), gpt_config.weighted_residual_path_init))
            self.mlp_residual_scale = nn.Parameter(torch.full((1,), gpt_config.weighted_residual_path_init))
        if self.use_weighted_main_path:
            self.attn_main_scale = nn.Parameter(torch.full((1,), gpt_config.weighted_main_path_init))
            self.mlp_main_scale = nn.Parameter(torch.full((1,), gpt_config.weighted_main_path_init))
        if not (self.use_weighted_residual_path or self.use_weighted_main_path):
            self.residual_scale = nn.Parameter(torch.full((1,), (2 * gpt_config.n_layers) ** -0.5), requires_grad=False)
        self.ln_1 = make_norm(gpt_config)
        attn_cls = MLAttention if gpt_config.use_mla else SelfAttention
        self.attn = attn_cls(gpt_config, training_config, layer_idx=layer_idx)
        self.ln_2 = make_norm(gpt_config)
        if self.use_moe:
            self.mlp = MoE(gpt_config, training_config, num_experts=gpt_config.num_experts,
                           top_k=gpt_config.moe_top_k, ep_rank=ep_rank, ep_size=ep_size)
        else:
            self.mlp = MLP(gpt_config, training_config)

    def _scales(self, which: str) -> Tuple[Optional[Tensor], Tensor]:
        """(alpha or None, beta) for 'attn' or 'mlp'."""
        if self.use_weighted_residual_path or self.use_weighted_main_path:
            alpha = getattr(self, f"{which}_residual_scale") if self.use_weighted_residual_path else None
            beta = getattr(self, f"{which}_main_scale") if self.use_weighted_main_path else None
            return alpha, beta
        return None, self.residual_scale

    @staticmethod
    def _mix(x: Tensor, branch: Tensor, alpha: Optional[Tensor], beta: Optional[Tensor]) -> Tensor:
        res = x if alpha is None else alpha * x
        return res + (branch if beta is None else beta * branch)

    def forward_prenormed(self, x: Tensor, h: Tensor, ctx: AttentionContext, next_norm: nn.Module, next_is_mxfp8: bool = False
                          ) -> Tuple[Tensor, Tensor, Optional[Tensor]]:
        """Block step for a chain of RMSNorm blocks: `h` is ln_1(x) computed by the previous link; every
        residual update is fused with the norm that follows it (the next block's ln_1, or the final norm).
        `next_is_mxfp8`: the consumer of the returned normalised rows is an MXFP8 projection (the norm kernel then emits
        their quantised copy too).  Returns (x_out, next_norm(x_out), balance_loss)."""
        alpha, beta = self._scales("attn")
        x, h2 = api.residual_rms_norm(x, self.attn(h, ctx), alpha, beta, self.ln_2.weight, norm_eps(self.ln_2, x.dtype))
        out = self.mlp(h2)
        balance = None
        if self.use_moe:
            out, balance = out
        alpha, beta = self._scales("mlp")
        x, h_next = api.residual_rms_norm(x, out, alpha, beta, next_norm.weight, norm_eps(next_norm, x.dtype), next_is_mxfp8)
        return x, h_next, balance

    def forward(self, x: Tensor, ctx: AttentionContext) -> Tuple[Tensor, Optional[Tensor]]:
        alpha, beta = self._scales("attn")
        x = self._mix(x, self.attn(apply_norm(self.ln_1, x), ctx), alpha, beta)
        out = self.mlp(apply_norm(self.ln_2, x))
        balance = None
        if self.use_moe:
            out, balance = out
        alpha, beta = self._scales("mlp")
        return self._mix(x, out, alpha, beta), balance
