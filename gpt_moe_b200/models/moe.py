"""Dropless token-choice mixture of experts.

Router in fp32, top-k selection, Switch-style load-balance loss, then sort-by-expert grouped
expert computation and a gate-weighted combine — no capacity factor, no dropped tokens
(reference `model/feedforward/moe.py:21-134`).  Parameter layout is the reference's:
`router.weight [E, hidden]`, `experts.{e}.up_proj.weight`, `experts.{e}.down_proj.weight`.

New here: an optional always-on shared expert (`shared_expert`, its own width) and expert
parallelism — with `expert_parallel_size > 1` each rank holds `num_experts / ep` experts and the
tokens travel by a counted all-to-all (see `parallel/ep.py`); the module's parameters are then
only the local experts, named by their GLOBAL index so checkpoints stay in the unsharded layout.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch.nn as nn
from torch import Tensor

from ..ops import api
from .linear import Linear
from .mlp import MLP


class MoE(nn.Module):
    def __init__(self, gpt_config, training_config, num_experts: int, top_k: int = 2,
                 ep_rank: int = 0, ep_size: int = 1) -> None:
        super().__init__()
        assert num_experts % ep_size == 0, "expert_parallel_size must divide num_experts"
        self.num_experts, self.top_k = num_experts, top_k
        self.ep_rank, self.ep_size = ep_rank, ep_size
        self.experts_per_rank = num_experts // ep_size
        self.first_expert = ep_rank * self.experts_per_rank
        self.full_softmax_gating = gpt_config.moe_full_softmax_gating
        self.load_balance_weight = training_config.moe_load_balance_weight
        self.router = Linear(gpt_config.hidden_size, num_experts, role="router", bias=False)
        # keys are global expert indices: experts.{e}.up_proj.weight.  All experts are constructed so that the
        # initial weights do not depend on the sharding; `keep_local_experts()` drops the others after init.
        self.experts = nn.ModuleDict({str(e): MLP(gpt_config, training_config) for e in range(num_experts)})
        self.shared_expert = (MLP(gpt_config, training_config, hidden_dim=gpt_config.moe_shared_expert_hidden_dim)
                              if gpt_config.moe_shared_expert_hidden_dim > 0 else None)
        self.ep_group = None            # set by parallel.ep.attach_expert_parallel

    def keep_local_experts(self) -> None:
        for e in range(self.num_experts):
            if not self.first_expert <= e < self.first_expert + self.experts_per_rank:
                del self.experts[str(e)]

    def local_experts(self):
        return [self.experts[str(e)] for e in range(self.first_expert, self.first_expert + self.experts_per_rank)]

    def forward(self, x: Tensor) -> Tuple[Tensor, Optional[Tensor]]:
        shape = x.shape
        hidden = x.reshape(-1, shape[-1])
        logits = self.router(hidden)
        want_balance = bool(self.training and self.load_balance_weight > 0)
        top_idx, gates, balance = api.router(logits, self.top_k, self.full_softmax_gating, want_balance, self.num_experts)
        experts = self.local_experts()
        first = experts[0]
        args = dict(
            up_weights=[m.up_proj.weight for m in experts], down_weights=[m.down_proj.weight for m in experts],
            up_biases=None if first.up_proj.bias is None else [m.up_proj.bias for m in experts],
            down_biases=None if first.down_proj.bias is None else [m.down_proj.bias for m in experts],
            activation=first.activation_name, up_precision=first.up_proj.precision,
            down_precision=first.down_proj.precision)
        if self.ep_size > 1:
            from ..parallel.ep import expert_parallel_moe
            out = expert_parallel_moe(self, hidden, top_idx, gates, args)
        else:
            out = api.moe_experts(hidden, top_idx, gates, **args)
        if self.shared_expert is not None:
            out = out + self.shared_expert(hidden)
        return out.reshape(shape), balance
