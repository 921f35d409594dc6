"""Expert parallelism: experts sharded over ranks, tokens exchanged by a counted all-to-all.

The reference keeps every expert on every rank (`model/feedforward/moe.py:30`); this is new.
Semantics stay dropless: no capacity factor, every routed (token, slot) pair is computed.

Host path (this file, works on gloo and NCCL; it is the NCCL baseline of the fused kernels):
  1. stable sort of the M*k slots by GLOBAL expert id — experts of one rank are contiguous, so
     the sorted rows are already grouped by destination rank;
  2. all-to-all of the per-expert counts, then of the rows (exactly-sized splits);
  3. received rows are grouped by local expert and run through the local grouped expert op;
  4. the results travel back by the inverse all-to-all and are combined with the gates.
Gradients flow through the same exchanges in reverse (`_AllToAll.backward`).
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist
from torch import Tensor

from ..ops import api
from ..ops import reference as ref


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, send_splits: List[int], recv_splits: List[int], group) -> Tensor:
        ctx.group, ctx.send_splits, ctx.recv_splits = group, send_splits, recv_splits
        out = x.new_empty((sum(recv_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), recv_splits, send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, grad: Tensor):
        out = grad.new_empty((sum(ctx.send_splits),) + tuple(grad.shape[1:]))
        dist.all_to_all_single(out, grad.contiguous(), ctx.send_splits, ctx.recv_splits, group=ctx.group)
        return out, None, None, None


def attach_expert_parallel(model, group, fused: bool = False, capacity_factor: float = 0.0) -> None:
    """Give every MoE layer of `model` its expert-parallel process group.  `fused` selects the CUDA path whose dispatch and
    combine kernels store / load rows directly in the peers' memory (`parallel.ep_fused`); it needs symmetric memory."""
    from ..models.moe import MoE
    for module in model.modules():
        if isinstance(module, MoE):
            module.ep_group = group
            module.ep_fused = fused
            module.ep_capacity_factor = capacity_factor


def expert_parallel_moe(moe, hidden: Tensor, top_idx: Tensor, gates: Tensor, args: dict) -> Tensor:
    from . import ep_fused
    if ep_fused.supported(moe, hidden):
        return ep_fused.fused_expert_parallel_moe(moe, hidden, top_idx, gates, args)
    group, ep, per_rank = moe.ep_group, moe.ep_size, moe.experts_per_rank
    top_k = top_idx.shape[1]
    _, order, inverse, offsets = ref.counted_expert_routing(top_idx, moe.num_experts)
    counts = torch.diff(offsets.to(torch.int64), prepend=offsets.new_zeros(1, dtype=torch.int64))
    send_counts = counts.view(ep, per_rank)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=group)
    send_splits = send_counts.sum(dim=1).tolist()
    recv_splits = recv_counts.sum(dim=1).tolist()

    packed = hidden[order // top_k]
    received = _AllToAll.apply(packed, send_splits, recv_splits, group)
    # received rows: for each source rank, its rows for local expert 0, 1, ... in that order
    local_expert = torch.repeat_interleave(
        torch.arange(per_rank, device=hidden.device).repeat(ep), recv_counts.reshape(-1))
    ones = torch.ones(received.shape[0], 1, dtype=gates.dtype, device=hidden.device)
    computed = api.moe_experts(received, local_expert[:, None], ones, **args)
    returned = _AllToAll.apply(computed, recv_splits, send_splits, group)
    return ref.combine_expert_outputs(returned, inverse, gates).to(hidden.dtype)
