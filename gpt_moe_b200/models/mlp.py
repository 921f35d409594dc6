"""Dense feed-forward block; also the parameter container of one MoE expert.

up -> activation -> down with gelu / relu / relu^2 / silu / SwiGLU.  SwiGLU's `up_proj` is
`[2*hidden_dim, hidden]` with the gate in the first half; "fair" SwiGLU shrinks `hidden_dim` to
round(2/3 * mlp_hidden_dim) so the parameter count matches the ungated variants
(reference `model/feedforward/mlp.py:16-75`).
"""
from __future__ import annotations

import torch.nn as nn
from torch import Tensor

from ..ops import api
from .linear import Linear


class MLP(nn.Module):
    def __init__(self, gpt_config, training_config, hidden_dim: int | None = None) -> None:
        super().__init__()
        self.activation_name = gpt_config.activation.lower()
        base = gpt_config.mlp_hidden_dim if hidden_dim is None else hidden_dim
        if self.activation_name == "swiglu":
            self.hidden_dim = round((2.0 / 3.0) * base) if (gpt_config.use_fair_swiglu and hidden_dim is None) else base
            up_width = 2 * self.hidden_dim
        else:
            self.hidden_dim = base
            up_width = self.hidden_dim
        self.up_proj = Linear(gpt_config.hidden_size, up_width, role="up_proj", bias=gpt_config.use_bias)
        self.down_proj = Linear(self.hidden_dim, gpt_config.hidden_size, role="down_proj", bias=gpt_config.use_bias)

    def activate(self, x: Tensor) -> Tensor:
        return api.activate(x, self.activation_name)

    def forward(self, x: Tensor) -> Tensor:
        return self.down_proj(self.activate(self.up_proj(x)))
