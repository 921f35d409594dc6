"""GPU data-parallel engine: flat symmetric buffers and optimizer kernels fused with their collectives.

Memory plan (per GPU; "symmetric" = allocated at the same offset on every rank and mapped into every rank, so a
kernel reaches a peer's copy by adding a per-rank byte delta to its own pointer):

  grad_muon   fp32 symmetric   weight gradients of all Muon matrices; the weight-gradient GEMMs write here directly
                               (`param.main_grad`), accumulating over micro-steps by TMA reduce-add
  compute     bf16 symmetric   GEMM operands ("compute copies") of all Muon matrices (`param.compute`); q/k/v of a
                               layer and the experts of a layer are adjacent, so the fused QKV GEMM and the grouped
                               expert GEMMs read plain views — no per-step cast, cat or stack
  adamw_param fp32 symmetric   every AdamW parameter (embeddings, LM head, norms, scalars); `param.data` are views
  adamw_grad  fp32 symmetric   their gradients; `param.grad` are views (autograd accumulates in place)
  masters     fp32 local       Muon master weights stay ordinary tensors; only the owner's copy is kept current

One optimizer step (`step()`), three kernels per bucket of same-shape matrices plus two barriers:
  barrier -> rs_muon_prepare (owner sums the gradient out of every rank's buffer + momentum/Nesterov/bf16 pack)
          -> Polar Express on tcgen05 GEMMs -> muon_apply_push (master update + bf16 copy stored to every rank)
          -> adamw_sharded (slice owner: sum gradients, AdamW, store new values to every rank) -> barrier
Each matrix has exactly one owner (balanced by orthogonalisation cost), so Muon's work is divided by the world
size instead of being repeated on every rank as in the reference (`optimizers/muon.py:147-224`), and gradients cross
NVLink once as reads (reduce-scatter) and weights once as bf16 stores (all-gather).  Expert weights under expert
parallelism are rank-local: owned locally, never reduced, never pushed.

With one GPU the same code runs with a world of one (no peers); the flat buffers still remove every per-step cast.
If symmetric memory cannot be set up the engine falls back to `CudaHostEngine` (NCCL collectives).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from . import dist_utils as du
from .ddp_engine import HostEngine, assign_owners, polar_cost, _to_cpu


class CudaHostEngine(HostEngine):
    """NCCL collectives + this framework's kernels for everything on-device: the measured NCCL baseline."""

    def forward_backward(self, model, x, y, document_ids, loss_scale: float, last_micro_step: bool):
        from ..ops import cuda_ops
        cuda_ops.set_loss_scale(loss_scale)
        return super().forward_backward(model, x, y, document_ids, loss_scale, last_micro_step)

    def step(self) -> None:
        from ..ops import cuda_ops
        super().step()
        cuda_ops.mark_parameters_updated()
        cuda_ops.check_status_deferred()                  # no host synchronisation per step; a failed step is reported at the next one


class SymmetricBuffer:
    """A flat tensor that every rank of `group` can address: `deltas[r]` is rank r's base minus this rank's base."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group=None) -> None:
        self.world = du.world_size(group)
        self.rank = du.get_rank(group)
        numel = max(int(numel), 4)
        self.handle = None
        if self.world == 1:
            self.tensor = torch.zeros(numel, dtype=dtype, device=device)
            self._deltas = [0]
            return
        import torch.distributed._symmetric_memory as symm
        self.tensor = symm.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm.rendezvous(self.tensor, group=group if group is not None else dist.group.WORLD)
        base = int(self.handle.buffer_ptrs[self.rank])
        self._deltas = [int(ptr) - base for ptr in self.handle.buffer_ptrs]

    def barrier(self) -> None:
        """All ranks' earlier work on the current streams is complete and visible before any rank continues."""
        if self.handle is not None and not self.dry_run:
            self.handle.barrier(channel=0)

    # Timing aid: with `dry_run` every "peer" offset points at this rank's own buffer and barriers are skipped, so a step
    # does the same arithmetic and moves the same bytes through local HBM instead of NVLink.  The difference between a
    # normal and a dry step is the communication time that is exposed (not hidden behind compute).  Results are wrong by
    # construction (each rank sees only its own gradients); use it for measurement only.
    dry_run = False

    @property
    def deltas(self) -> List[int]:
        return [0] * len(self._deltas) if self.dry_run else self._deltas


def _aligned(n: int, multiple: int = 64) -> int:
    return (n + multiple - 1) // multiple * multiple


class FusedEngine:
    def __init__(self, model: nn.Module, training_config, optimizers: Dict[str, torch.optim.Optimizer],
                 dp_group=None, ep_size: int = 1, ep_group=None) -> None:
        self.model, self.cfg, self.optimizers = model, training_config, optimizers
        self.group = dp_group
        self.world, self.rank = du.world_size(dp_group), du.get_rank(dp_group)
        self.ep_size, self.ep_group = ep_size, ep_group
        self.device = next(model.parameters()).device
        if getattr(training_config, "grad_reduce_dtype", "fp32") != "fp32":
            raise NotImplementedError("gradients are reduced in fp32 (grad_reduce_dtype must be 'fp32')")
        groups = model.optimizer_param_groups()
        named = dict(model.named_parameters())
        muon_names = [n for n, _ in groups["muon"]]
        expert_local = {n for n in muon_names if ".mlp.experts." in n} if ep_size > 1 else set()
        self.small = [(n, named[n]) for n in muon_names if min(named[n].shape) < 128 or named[n].shape[1] % 8 or named[n].shape[0] % 8]
        small_names = {n for n, _ in self.small}
        self.big = [(n, named[n]) for n in self._layout_order(muon_names) if n not in small_names]
        self.adamw_named = groups["adamw_decay"] + groups["adamw_nodecay"]
        decay_names = {n for n, _ in groups["adamw_decay"]}
        wd = optimizers["adamw"].param_groups[0]["weight_decay"]

        # ---- flat buffers -----------------------------------------------------------------------------------------
        self.big_offsets: Dict[str, int] = {}
        cursor = 0
        for n, p in self.big + self.small:
            self.big_offsets[n] = cursor
            cursor += _aligned(p.numel())
        self.small_range = (self.big_offsets[self.small[0][0]], cursor) if self.small else (0, 0)
        self.grad_muon = SymmetricBuffer(cursor, torch.float32, self.device, dp_group)
        self.compute = SymmetricBuffer(cursor, torch.bfloat16, self.device, dp_group)
        self.adamw_offsets: Dict[str, int] = {}
        cursor = 0
        for n, p in self.adamw_named:
            self.adamw_offsets[n] = cursor
            cursor += _aligned(p.numel())
        self.adamw_numel = _aligned(cursor, 4 * max(self.world, 1))
        self.adamw_param = SymmetricBuffer(self.adamw_numel, torch.float32, self.device, dp_group)
        self.adamw_grad = SymmetricBuffer(self.adamw_numel, torch.float32, self.device, dp_group)
        self.adamw_decay = torch.zeros(self.adamw_numel, dtype=torch.float32, device=self.device)

        for n, p in self.big + self.small:
            off = self.big_offsets[n]
            p.main_grad = self.grad_muon.tensor[off: off + p.numel()].view(p.shape)
            p.compute = self.compute.tensor[off: off + p.numel()].view(p.shape)
            p.grad_ready = False
        for n, p in self.adamw_named:
            off = self.adamw_offsets[n]
            view = self.adamw_param.tensor[off: off + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.grad = self.adamw_grad.tensor[off: off + p.numel()].view(p.shape)
            if p.dim() == 2:                          # GEMM weights (LM head): weight-gradient GEMMs write the flat buffer directly
                p.main_grad = p.grad
                p.grad_ready = True                   # the buffer is zeroed every step, so the GEMM always accumulates
            if n in decay_names:
                self.adamw_decay[off: off + p.numel()] = wd
        self.refresh_from_parameters()

        # ---- ownership ------------------------------------------------------------------------------------------------
        shared = [(n, p) for n, p in self.big if n not in expert_local]
        self.owners = assign_owners(shared, self.world, lambda p: polar_cost(p.shape)) if self.world > 1 else {n: 0 for n, _ in shared}
        self.owned_shared = [(n, p) for n, p in shared if self.owners[n] == self.rank]
        self.owned_local = [(n, p) for n, p in self.big if n in expert_local]
        per = self.adamw_numel // self.world
        self.adamw_lo = self.rank * per
        self.adamw_n = per
        moment_dtype = optimizers["adamw"].moment_dtype
        self.adamw_m = torch.zeros(per, dtype=moment_dtype, device=self.device)
        self.adamw_v = torch.zeros(per, dtype=moment_dtype, device=self.device)
        self.adamw_step = 0
        self._import_optimizer_state()

        # ---- overlap of the Muon reduce / update / push with the backward pass ---------------------------------------------
        # When the backward of a transformer block has been issued, this rank publishes a flag for that block; on a second
        # stream the owner of a matrix waits (bounded) for the block's flags of all ranks and then runs reduce + momentum +
        # Polar Express + push for its matrices of that block while the main stream continues with the earlier blocks.
        self.overlap = bool(self.world > 1 and getattr(training_config, "overlap_grad_reduce", False))
        self.layer_items: Dict[int, List[Tuple[str, nn.Parameter]]] = {}
        for n, p in self.owned_shared:
            parts = n.split(".")
            layer = int(parts[2]) if len(parts) > 2 and parts[1] == "h" and parts[2].isdigit() else -1
            self.layer_items.setdefault(layer, []).append((n, p))
        n_slots = max([layer for layer in self.layer_items] + [0]) + 2
        self.flags = SymmetricBuffer(n_slots * max(self.world, 1), torch.int32, self.device, dp_group) if self.overlap else None
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.overlap else None
        self.step_counter = 0
        self._early_layers: set = set()
        # ---- CUDA graphs: forward + backward of one micro-step, captured per (input shape, window, loss scale) ----------------
        self.use_graphs = bool(getattr(training_config, "use_cuda_graphs", True) and self.device.type == "cuda")
        self._graphs: Dict[tuple, dict] = {}
        self._barrier()

    # ---- layout helpers ---------------------------------------------------------------------------------------------------
    @staticmethod
    def _layout_order(names: Sequence[str]) -> List[str]:
        """Model order, except that inside a layer all expert up-projections are adjacent and all down-projections are
        adjacent (they are read as one [E, N, K] stack), and q/k/v stay adjacent (one fused GEMM operand)."""
        def key(name: str):
            parts = name.split(".")
            layer = int(parts[2]) if len(parts) > 2 and parts[1] == "h" else -1
            if ".mlp.experts." in name:
                expert = int(parts[parts.index("experts") + 1])
                kind = 0 if "up_proj" in name else 1
                return (layer, 2, kind, expert)
            order = {"q_proj": 0, "k_proj": 1, "v_proj": 2, "out_proj": 3}
            for k, v in order.items():
                if k in name:
                    return (layer, 0, v, 0)
            return (layer, 1, 0, 0)
        indexed = {n: i for i, n in enumerate(names)}
        return sorted(names, key=lambda n: key(n) + (indexed[n],))

    def _barrier(self) -> None:
        self.grad_muon.barrier()

    def set_comm_dry_run(self, enabled: bool) -> None:
        """Measurement mode: peer offsets collapse onto this rank and barriers are skipped (see `SymmetricBuffer.dry_run`)."""
        for buf in (self.grad_muon, self.compute, self.adamw_param, self.adamw_grad):
            buf.dry_run = enabled

    def refresh_from_parameters(self) -> None:
        """Rebuild the bf16 GEMM copies from the fp32 masters (after construction, a checkpoint load or a restore)."""
        from ..ops import cuda_ops
        for _, p in self.big + self.small:
            cuda_ops._cast_into(p.data, p.compute)
        cuda_ops.mark_parameters_updated()

    def _import_optimizer_state(self) -> None:
        """Adopt state loaded into the torch-layout optimizers (checkpoint resume): AdamW moments into this rank's slice."""
        adamw = self.optimizers["adamw"]
        steps = []
        for n, p in self.adamw_named:
            state = adamw.state.get(p)
            if not state:
                continue
            steps.append(int(round(float(state["step"]))))
            off = self.adamw_offsets[n]
            lo, hi = max(off, self.adamw_lo), min(off + p.numel(), self.adamw_lo + self.adamw_n)
            if lo < hi:
                self.adamw_m[lo - self.adamw_lo: hi - self.adamw_lo] = state["exp_avg"].reshape(-1)[lo - off: hi - off].to(self.adamw_m.dtype)
                self.adamw_v[lo - self.adamw_lo: hi - self.adamw_lo] = state["exp_avg_sq"].reshape(-1)[lo - off: hi - off].to(self.adamw_v.dtype)
            adamw.state.pop(p, None)
        if steps:
            self.adamw_step = max(steps)

    def snapshot(self) -> dict:
        """State that lives outside the torch optimizers (used by the kernel warm-up to restore exactly)."""
        return {"m": self.adamw_m.clone(), "v": self.adamw_v.clone(), "step": self.adamw_step}

    def restore(self, snap: dict) -> None:
        self.adamw_m.copy_(snap["m"])
        self.adamw_v.copy_(snap["v"])
        self.adamw_step = snap["step"]
        self.refresh_from_parameters()

    # ---- step protocol --------------------------------------------------------------------------------------------------------
    def zero_grad(self) -> None:
        self.adamw_grad.tensor.zero_()
        for _, p in self.big + self.small:
            p.grad_ready = False
            p.grad = None

    def _graph_eligible(self, model, x, document_ids) -> bool:
        """Graph replay needs a step whose launches do not depend on host-side state: one micro-step per step (the
        first-write / accumulate choice of the weight-gradient GEMMs is then fixed), no expert-parallel exchange (its barriers
        and peer stores stay eager), no document ids, the plain chain of blocks (no activation checkpointing or offloading)."""
        raw = self.model
        return (self.use_graphs and x.is_cuda and document_ids is None and self.cfg.grad_accum_mini_steps == 1 and self.ep_size == 1
                and not self.overlap and raw.training and torch.is_grad_enabled()
                and not getattr(raw, "use_activation_checkpointing", False) and getattr(raw, "activation_offloader", None) is None)

    def _graphed_forward_backward(self, model, x, y, loss_scale: float):
        """Third and later calls with the same key replay a captured graph of forward + backward (inputs are copied into the
        graph's static tensors; losses come back in static tensors); the first two run eagerly (they also warm every cache)."""
        from ..ops import cuda_ops
        window = getattr(getattr(self.model, "sliding_window_size", None), "host_value", None)
        key = (tuple(x.shape), tuple(y.shape), window, float(loss_scale), x.dtype)
        entry = self._graphs.setdefault(key, {"calls": 0})
        entry["calls"] += 1
        if "graph" not in entry:
            if entry["calls"] <= 2:
                return None
            torch.cuda.synchronize()
            sx, sy = x.clone(), y.clone()
            graph = torch.cuda.CUDAGraph()
            before = cuda_ops.launch_count()
            try:
                with torch.cuda.graph(graph):
                    loss, token_loss, balance = model(sx, sy, document_ids=None)
                    (loss * loss_scale).backward()
            except Exception as exc:              # capture refused (an op that cannot be captured): stay eager from now on
                self.use_graphs = False
                self._graphs.clear()
                torch.cuda.synchronize()
                import sys
                print(f"CUDA graph capture of the training step failed ({type(exc).__name__}: {exc}); continuing without graphs",
                      file=sys.stderr)
                return None
            entry.update(graph=graph, x=sx, y=sy, outs=(loss.detach(), token_loss.detach(), balance.detach()),
                         launches=cuda_ops.launch_count() - before)
            # a captured step keeps its activations alive in the graph's memory pool: when a schedule moves on (new window,
            # new batch size) only the two most recent graphs are kept
            captured = [k for k, e in self._graphs.items() if "graph" in e]
            for stale in captured[:-2]:
                del self._graphs[stale]
            # the capture only recorded the launches: the replay below is what computes this step
        else:
            entry["x"].copy_(x, non_blocking=True)
            entry["y"].copy_(y, non_blocking=True)
        entry["graph"].replay()
        cuda_ops.add_launches(entry["launches"])
        return entry["outs"]

    def forward_backward(self, model, x, y, document_ids, loss_scale: float, last_micro_step: bool):
        from ..ops import cuda_ops
        cuda_ops.set_loss_scale(loss_scale)
        if self._graph_eligible(model, x, document_ids):
            outs = self._graphed_forward_backward(model, x, y, loss_scale)
            if outs is not None:
                return outs
        early = self.overlap and last_micro_step and self.optimizers.get("muon") is not None
        if early:
            self.step_counter += 1
            self._early_layers = set()
        self.model.block_grad_hook = self._on_block_backward if early else None
        try:
            loss, token_loss, balance = model(x, y, document_ids=document_ids)
            (loss * loss_scale).backward()
        finally:
            self.model.block_grad_hook = None
        return loss, token_loss, balance

    def _on_block_backward(self, layer: int) -> None:
        """Called from the backward pass once every gradient of block `layer` has been issued on the current stream."""
        from ..ops import cuda_ops
        c = cuda_ops.ext()
        if layer in self._early_layers:
            return
        self._early_layers.add(layer)
        c.flag_signal(self.flags.tensor, self.flags.deltas, layer * self.world + self.rank, self.step_counter)
        items = self.layer_items.get(layer)
        if not items:
            return
        ready = torch.cuda.Event()
        ready.record()
        g = self.optimizers["muon"].param_groups[0]
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ready)
            c.flag_wait(self.flags.tensor, layer * self.world, self.world, self.step_counter)
            self._muon_update(items, self.grad_muon.deltas, self.compute.deltas, g["lr"], g["momentum"], g["nesterov"])

    def _muon_buckets(self, items: List[Tuple[str, nn.Parameter]]):
        buckets: Dict[Tuple[int, int], List[nn.Parameter]] = {}
        for _, p in items:
            rows, cols = p.shape
            if rows == 3 * cols:                      # fused (3d, d) projections are orthogonalised as three squares
                raise NotImplementedError("fused (3d, d) matrices are not laid out by this engine")
            buckets.setdefault((rows, cols), []).append(p)
        return buckets

    def _muon_update(self, items, deltas_grad: List[int], deltas_compute: List[int], lr: float, momentum: float, nesterov: bool,
                     max_batch: int = 128) -> None:
        from ..ops import cuda_ops
        c = cuda_ops.ext()
        muon = self.optimizers["muon"]
        for (rows, cols), params in self._muon_buckets(items).items():
            tall = rows > cols
            m, k = (cols, rows) if tall else (rows, cols)
            alpha = -lr * max(rows, cols) ** 0.5
            for start in range(0, len(params), max_batch):
                batch = params[start: start + max_batch]
                bufs = []
                for p in batch:
                    state = muon.state[p]
                    if "momentum_buffer" not in state:
                        state["momentum_buffer"] = torch.zeros_like(p.data)
                    bufs.append(state["momentum_buffer"])
                packed = torch.empty((len(batch), m, k), dtype=torch.bfloat16, device=self.device)
                sumsq = torch.zeros(len(batch), dtype=torch.float32, device=self.device)
                c.rs_muon_prepare(cuda_ops._ptr_table([p.main_grad for p in batch]), cuda_ops._ptr_table(bufs), packed, sumsq,
                                  rows, cols, cols, cols, momentum, nesterov, tall, deltas_grad, normalize=False)
                update = cuda_ops.polar_express_bf16(packed, sumsq)      # the first iteration's epilogues apply the normalisation
                c.muon_apply_push(cuda_ops._ptr_table([p.data for p in batch]), cuda_ops._ptr_table([p.compute for p in batch]),
                                  update, rows, cols, cols, cols, alpha, tall, deltas_compute)

    def step(self) -> None:
        from ..ops import cuda_ops
        from ..ops import reference as ref
        c = cuda_ops.ext()
        muon, adamw = self.optimizers.get("muon"), self.optimizers["adamw"]
        self._barrier()                                   # every rank's gradients are complete
        if muon is not None:
            g = muon.param_groups[0]
            lr, momentum, nesterov = g["lr"], g["momentum"], g["nesterov"]
            if g["backend"] != "polarexpress":
                raise NotImplementedError("the fused engine implements the Polar Express backend")
            remaining = self.owned_shared
            if self._early_layers:
                # blocks whose update already ran beside the backward pass: join that stream, then do what is left
                torch.cuda.current_stream().wait_stream(self.comm_stream)
                remaining = [(n, p) for layer, items in self.layer_items.items() if layer not in self._early_layers for n, p in items]
                self._early_layers = set()
            self._muon_update(remaining, self.grad_muon.deltas, self.compute.deltas, lr, momentum, nesterov)
            self._muon_update(self.owned_local, [0], [0], lr, momentum, nesterov)
            # (issued after the large batches: its many tiny launches are host-bound and hide behind the queued GEMMs)
            # tiny matrices (routers): every rank averages them out of all buffers and repeats the small update
            if self.small:
                lo, hi = self.small_range
                local = self.grad_muon.tensor[lo:hi]
                if self.world > 1 and not self.grad_muon.dry_run:
                    total = torch.zeros_like(local)
                    for r in range(self.world):
                        total += self.grad_muon.handle.get_buffer(r, (hi - lo,), torch.float32, lo)
                    local = total / self.world
                grads, bufs = [], []
                for n, p in self.small:
                    off = self.big_offsets[n] - lo
                    state = muon.state[p]
                    if "momentum_buffer" not in state:
                        state["momentum_buffer"] = torch.zeros_like(p.data)
                    buf = state["momentum_buffer"]
                    gflat = local[off: off + p.numel()].view(p.shape)
                    buf.mul_(momentum).add_(gflat)
                    grads.append(gflat.add(buf, alpha=momentum) if nesterov else buf)
                shapes: Dict[tuple, List[int]] = {}
                for i, (_, p) in enumerate(self.small):
                    shapes.setdefault(tuple(p.shape), []).append(i)
                for shape, idxs in shapes.items():
                    o = ref.polar_express(torch.stack([grads[i] for i in idxs]))
                    for i, oi in zip(idxs, o):
                        p = self.small[i][1]
                        p.data.add_(oi.to(p.dtype), alpha=-lr * max(shape) ** 0.5)
                        p.compute.copy_(p.data)
        g0 = adamw.param_groups[0]
        self.adamw_step += 1
        c.adamw_sharded(self.adamw_param.tensor, self.adamw_grad.tensor, self.adamw_m, self.adamw_v, self.adamw_decay,
                        self.adamw_lo, self.adamw_n, g0["lr"], g0["betas"][0], g0["betas"][1], g0["eps"], self.adamw_step,
                        self.adamw_grad.deltas, self.adamw_param.deltas)
        self._barrier()                                   # every rank's pushes have landed
        cuda_ops.mark_parameters_updated()
        cuda_ops.check_status_deferred()                  # no host synchronisation per step; a failed step is reported at the next one

    # ---- checkpoint helpers -------------------------------------------------------------------------------------------------------
    def sync_masters(self) -> None:
        """Bring every rank's fp32 Muon masters up to date from their owners (needed only before saving or exporting)."""
        if self.world == 1:
            return
        for owner in range(self.world):
            mine = [p for n, p in self.big if self.owners.get(n, -1) == owner]
            if not mine:
                continue
            flat = torch.cat([p.data.reshape(-1) for p in mine])
            dist.broadcast(flat, src=owner, group=self.group)
            if owner != self.rank:
                off = 0
                for p in mine:
                    p.data.copy_(flat[off: off + p.numel()].view_as(p))
                    off += p.numel()

    def full_model_state(self) -> Dict[str, Tensor]:
        from ..checkpointing.checkpoint import gather_full_state_dict
        self.sync_masters()
        return gather_full_state_dict(self.model, self.ep_group)

    def full_optimizer_state_dicts(self) -> Dict[str, dict]:
        """Optimizer state in the replicated torch layout (per-parameter `momentum_buffer`; `step`, `exp_avg`, `exp_avg_sq`)."""
        out: Dict[str, dict] = {}
        adamw = self.optimizers["adamw"]
        m_full = torch.empty(self.adamw_numel, dtype=self.adamw_m.dtype, device=self.device)
        v_full = torch.empty_like(m_full)
        if self.world > 1:
            dist.all_gather_into_tensor(m_full, self.adamw_m, group=self.group)
            dist.all_gather_into_tensor(v_full, self.adamw_v, group=self.group)
        else:
            m_full.copy_(self.adamw_m)
            v_full.copy_(self.adamw_v)
        index = {id(p): i for i, p in enumerate(q for g in adamw.param_groups for q in g["params"])}
        state = {}
        for n, p in self.adamw_named:
            off = self.adamw_offsets[n]
            state[index[id(p)]] = {"step": torch.tensor(float(self.adamw_step)),
                                   "exp_avg": m_full[off: off + p.numel()].view(p.shape).cpu().clone(),
                                   "exp_avg_sq": v_full[off: off + p.numel()].view(p.shape).cpu().clone()}
        out["adamw"] = {"state": dict(sorted(state.items())), "param_groups": adamw.state_dict()["param_groups"]}
        if "muon" in self.optimizers:
            sd = self.optimizers["muon"].state_dict()
            local_state = {k: _to_cpu(v) for k, v in sd["state"].items()}
            if self.world > 1:
                parts: List[Optional[dict]] = [None] * self.world
                dist.all_gather_object(parts, local_state, group=self.group)
                merged: dict = {}
                for part in parts:
                    for k, v in part.items():
                        merged.setdefault(k, v)
                local_state = merged
            out["muon"] = {"state": dict(sorted(local_state.items())), "param_groups": sd["param_groups"]}
        return out


def build_cuda_engine(model, training_config, optimizers, ep_size: int = 1, ep_group=None):
    """The fused engine when the model fits its assumptions (fp32 masters, Polar Express Muon, peer-mappable memory);
    otherwise the NCCL engine."""
    usable = (training_config.use_fused_collectives and "muon" in optimizers
              and optimizers["muon"].param_groups[0]["backend"] == "polarexpress"
              and all(p.dtype == torch.float32 for p in model.parameters())
              and not any(p.shape[0] == 3 * p.shape[1] for p in model.parameters() if p.dim() == 2))
    if usable:
        try:
            return FusedEngine(model, training_config, optimizers, dp_group=None, ep_size=ep_size, ep_group=ep_group)
        except Exception as exc:  # symmetric memory unavailable on this machine
            if du.get_rank() == 0:
                import sys
                print(f"fused engine unavailable ({type(exc).__name__}: {exc}); using NCCL collectives", file=sys.stderr)
    return CudaHostEngine(model, training_config, optimizers, dp_group=None, ep_size=ep_size)
