"""Role-tagged linear layer.

Every projection in the model is a `Linear` carrying a `role` (q_proj, k_proj, v_proj, out_proj,
up_proj, down_proj, router, lm_head) whose `precision`/`backend` are switched per phase by
`GPT.set_precision_phase` (reference `model/linear/linear.py:10-23`, `model/gpt.py:195-203`).

precision "default": the GEMM runs in the activation dtype (bf16 on the GPU, fp32 on CPU).
precision "mxfp8" / "fp8": e4m3 operands with one E8M0 power-of-two scale per 32 elements along
the contraction dimension, fp32 accumulation.  On CPU this is emulated exactly by
`ops.reference.mxfp8_linear` so that the GPU kernel has an oracle.
"""
from __future__ import annotations

import torch.nn as nn
from torch import Tensor

from ..ops import api


class Linear(nn.Linear):
    def __init__(self, in_features: int, out_features: int, *, role: str, bias: bool = True) -> None:
        super().__init__(in_features, out_features, bias=bias)
        self.role = role
        self.precision = "default"
        self.backend = "custom"

    def forward(self, x: Tensor) -> Tensor:
        return api.linear(x, self.weight, self.bias, self.precision)
