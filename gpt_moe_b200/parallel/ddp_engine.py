"""Data-parallel engine: gradient synchronisation, sharded optimizer step, parameter sync.

This replaces `torch.nn.parallel.DistributedDataParallel` + replicated optimizers of the
reference (`train.py:213-236, 481-490`) with one object that owns the whole
"backward -> reduce -> update -> broadcast" pipeline:

* parameters are partitioned among ranks by whole tensor ("owners"), balanced by the
  orthogonalisation cost for Muon matrices and by size for AdamW tensors;
* gradients are reduced so that each owner holds the averaged gradient of what it owns
  (reduce-scatter by ownership), the owner applies the optimizer update (sharded Muon / AdamW),
  and the updated parameters are all-gathered.  The reference all-reduces every gradient and then
  repeats the full optimizer computation on every rank (`optimizers/muon.py:147-224`);
* expert parameters under expert parallelism are never reduced across the expert-parallel group
  (each rank holds different experts) — only across replicas of the same expert, if any.

Two implementations share this interface.  `HostEngine` (this file) uses `torch.distributed`
collectives and works on CPU/gloo and on CUDA/NCCL — it is the measured NCCL baseline.
`parallel/fused_engine.py` runs the same plan through peer-memory kernels.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from . import dist_utils as du


def polar_cost(shape: Sequence[int]) -> float:
    """FLOPs of five Polar Express iterations on a matrix (fused 3d x d counted as three squares)."""
    rows, cols = int(shape[0]), int(shape[1])
    if rows == 3 * cols:
        return 3 * polar_cost((cols, cols))
    m, n = min(rows, cols), max(rows, cols)
    return 5.0 * (2 * m * m * n * 2 + 2 * m * m * m)


def assign_owners(named_params: List[Tuple[str, Tensor]], world: int, cost: Callable[[Tensor], float]) -> Dict[str, int]:
    """Greedy longest-processing-time partition; deterministic (ties broken by name) so every rank
    computes the same map without communicating."""
    loads = [0.0] * world
    owners: Dict[str, int] = {}
    for name, p in sorted(named_params, key=lambda kv: (-cost(kv[1]), kv[0])):
        r = min(range(world), key=lambda i: (loads[i], i))
        owners[name] = r
        loads[r] += cost(p)
    return owners


class HostEngine:
    """Gradient reduction + sharded optimizer step with `torch.distributed` collectives."""

    def __init__(self, model: nn.Module, training_config, optimizers: Dict[str, torch.optim.Optimizer],
                 dp_group=None, ep_size: int = 1, expert_replica_group=None) -> None:
        self.model = model
        self.cfg = training_config
        self.optimizers = optimizers
        self.group = dp_group
        self.world = du.world_size(dp_group)
        self.rank = du.get_rank(dp_group)
        self.ep_size = ep_size
        self.shard_optimizer = bool(training_config.shard_muon) and self.world > 1
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        self.expert_names = {n for n, _ in named if ".mlp.experts." in n} if ep_size > 1 else set()
        # replicas of one expert exist only when the expert-parallel group is smaller than the world: the ranks with the
        # same position in their expert-parallel group (rank % ep_size) hold the same experts and form a replica group
        self.expert_replicas = self.world // ep_size if ep_size > 1 else 1
        if self.expert_replicas > 1 and expert_replica_group is None:
            raise ValueError("expert_parallel_size smaller than the world size needs the expert replica group "
                             "(ranks with equal rank % expert_parallel_size)")
        self.expert_replica_group = expert_replica_group if self.expert_replicas > 1 else None
        self.dense = [(n, p) for n, p in named if n not in self.expert_names]
        self.experts = [(n, p) for n, p in named if n in self.expert_names]
        self.owners: Dict[str, int] = {}
        if self.shard_optimizer:
            groups = model.optimizer_param_groups()
            muon_names = {n for n, _ in groups["muon"]}
            muon = [(n, p) for n, p in self.dense if n in muon_names]
            other = [(n, p) for n, p in self.dense if n not in muon_names]
            self.owners.update(assign_owners(muon, self.world, lambda p: polar_cost(p.shape)))
            self.owners.update(assign_owners(other, self.world, lambda p: float(p.numel())))
            by_param = {id(p): self.owners[n] for n, p in self.dense}
            for opt in optimizers.values():
                if hasattr(opt, "owner_of"):
                    opt.owner_of = lambda p, _m=by_param: _m.get(id(p), self.rank) == self.rank
        self._owned_ids = {id(p) for n, p in self.dense if self.owners.get(n, self.rank) == self.rank}

    # ---- forward / backward -------------------------------------------------------------------------
    def forward_backward(self, model, x, y, document_ids, loss_scale: float, last_micro_step: bool):
        """One micro-step.  Gradients accumulate locally; reduction happens in `step()` (after the
        last micro-step), which is the `require_backward_grad_sync` rule of the reference (`train.py:415`)."""
        loss, token_loss, balance = model(x, y, document_ids=document_ids)
        (loss * loss_scale).backward()
        return loss, token_loss, balance

    # ---- gradient synchronisation ---------------------------------------------------------------
    def _flat_all_reduce(self, tensors: List[Tensor], group, world: int) -> None:
        if not tensors or world == 1:
            return
        bucket_bytes = self.cfg.grad_bucket_mb * 2 ** 20
        bucket: List[Tensor] = []
        size = 0

        def flush() -> None:
            nonlocal bucket, size
            if not bucket:
                return
            flat = torch.cat([t.reshape(-1) for t in bucket])
            dist.all_reduce(flat, group=group)
            flat /= world
            offset = 0
            for t in bucket:
                t.copy_(flat[offset: offset + t.numel()].view_as(t))
                offset += t.numel()
            bucket, size = [], 0

        for t in tensors:
            bucket.append(t)
            size += t.numel() * t.element_size()
            if size >= bucket_bytes:
                flush()
        flush()

    def reduce_gradients(self) -> None:
        """Average gradients over the data-parallel replicas (experts: over their replicas only)."""
        if self.world == 1:
            return
        for _, p in self.dense + self.experts:
            if p.grad is None:
                p.grad = torch.zeros_like(p)
        self._flat_all_reduce([p.grad for _, p in self.dense], self.group, self.world)
        if self.experts and self.expert_replicas > 1:
            self._flat_all_reduce([p.grad for _, p in self.experts], self.expert_replica_group, self.expert_replicas)

    # ---- optimizer step + parameter sync ----------------------------------------------------------
    def step(self) -> None:
        self.reduce_gradients()
        adamw = self.optimizers["adamw"]
        if self.shard_optimizer:
            # AdamW skips tensors whose .grad is None: hide the gradients this rank does not own
            hidden = []
            for _, p in self.dense:
                if id(p) not in self._owned_ids and p.grad is not None:
                    hidden.append((p, p.grad))
                    p.grad = None
            for opt in self.optimizers.values():
                opt.step()
            for p, g in hidden:
                p.grad = g
            self._broadcast_owned()
        else:
            for opt in self.optimizers.values():
                opt.step()

    def _broadcast_owned(self) -> None:
        """All-gather of updated parameters, expressed as one flat broadcast per owner."""
        for owner in range(self.world):
            mine = [p for n, p in self.dense if self.owners[n] == owner]
            if not mine:
                continue
            flat = torch.cat([p.data.reshape(-1) for p in mine])
            dist.broadcast(flat, src=dist.get_global_rank(self.group, owner) if self.group is not None else owner, group=self.group)
            if owner != self.rank:
                offset = 0
                for p in mine:
                    p.data.copy_(flat[offset: offset + p.numel()].view_as(p))
                    offset += p.numel()

    def zero_grad(self) -> None:
        for opt in self.optimizers.values():
            opt.zero_grad(set_to_none=True)

    # ---- checkpoint helpers ----------------------------------------------------------------------
    def contributes_state(self, name: str) -> bool:
        """Does this rank hand in the optimizer state of parameter `name` at save time?  Exactly one rank does: the owner of
        a sharded tensor (rank 0 when the optimizer is replicated), and for an expert its holder in the first
        expert-parallel group."""
        if name in self.expert_names:
            return self.rank < self.ep_size
        return self.owners.get(name, 0) == self.rank

    def drop_foreign_state(self) -> None:
        """After a resume every rank has loaded the full optimizer state; keep only what this rank updates, so that a stale
        copy of someone else's state can never be saved."""
        if not self.shard_optimizer:
            return
        foreign = {id(p) for n, p in self.dense if self.owners.get(n, self.rank) != self.rank}
        for opt in self.optimizers.values():
            for p in [p for p in opt.state if id(p) in foreign]:
                del opt.state[p]

    def full_optimizer_state_dicts(self) -> Dict[str, dict]:
        """Optimizer state dicts in the unsharded torch layout (collective): each entry comes from the one rank that
        `contributes_state` names, matched by parameter name and keyed by the unsharded model's parameter order."""
        from ..checkpointing.checkpoint import merge_optimizer_state
        return {name: merge_optimizer_state(self.model, opt, self.contributes_state, self.group)
                for name, opt in self.optimizers.items()}


def _to_cpu(obj):
    if isinstance(obj, Tensor):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    return obj
