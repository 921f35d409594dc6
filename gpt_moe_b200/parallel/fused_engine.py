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
parallelism belong to the rank that holds the expert: with as many expert-parallel ranks as ranks they are never reduced or
pushed; with fewer, the ranks that hold the same experts (equal `rank % expert_parallel_size`) each sum that expert's
gradient out of the replicas' buffers and repeat the identical update.

The barriers are `PeerBarrier`s: one small kernel per rank that publishes an epoch into every peer's flag table and polls
its own table with a cycle budget; a peer that never arrives makes the wait give up with status 601 (reported by
`cuda_ops.check_status_deferred`) instead of spinning for ever.  After status 601 the step's reductions ran on incomplete
gradients and their results were pushed to every rank: the only recovery is to restore from a checkpoint.

With one GPU the same code runs with a world of one (no peers); the flat buffers still remove every per-step cast.
If symmetric memory cannot be set up, building the engine raises; `training.allow_nccl_fallback=True` selects
`CudaHostEngine` (NCCL collectives) instead.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from . import dist_utils as du
from .ddp_engine import HostEngine, assign_owners, polar_cost


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
        torch.cuda.synchronize(device)        # the zeros are in place before the rendezvous lets any peer write here
        self.handle = symm.rendezvous(self.tensor, group=group if group is not None else dist.group.WORLD)
        base = int(self.handle.buffer_ptrs[self.rank])
        self._deltas = [int(ptr) - base for ptr in self.handle.buffer_ptrs]

    # Timing aid: with `dry_run` every "peer" offset points at this rank's own buffer and barriers are skipped, so a step
    # does the same arithmetic and moves the same bytes through local HBM instead of NVLink.  The difference between a
    # normal and a dry step is the communication time that is exposed (not hidden behind compute).  Results are wrong by
    # construction (each rank sees only its own gradients); use it for measurement only.
    dry_run = False

    @property
    def deltas(self) -> List[int]:
        return [0] * len(self._deltas) if self.dry_run else self._deltas


class PeerBarrier:
    """Device-side barrier over the ranks of `group`: `sync()` queues one kernel on the current stream that (1) publishes this
    rank's next epoch into its slot of every rank's flag table, after a system-scope fence, and (2) polls its own table until
    every rank's epoch has arrived, with a cycle budget (status 601 when it runs out).  The epoch counter lives on the device,
    so the launch is identical every time and can sit inside a CUDA graph."""

    def __init__(self, device, group=None) -> None:
        self.flags = SymmetricBuffer(max(du.world_size(group), 4), torch.int32, device, group)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.world, self.rank = self.flags.world, self.flags.rank
        self.dry_run = False
        if self.world > 1:
            torch.cuda.synchronize(device)
            dist.barrier(group=group)         # host-side, once: every rank's table and epoch word exist and are zero

    def sync(self, budget_cycles: int = 0) -> None:
        """All ranks' earlier work on their current streams is complete and visible before any rank's later work starts."""
        if self.world == 1 or self.dry_run:
            return
        from ..ops import cuda_ops
        cuda_ops.ext().peer_barrier(self.flags.tensor, self.flags._deltas, self.rank, self.epoch, budget_cycles)


def _aligned(n: int, multiple: int = 64) -> int:
    return (n + multiple - 1) // multiple * multiple


# matrices with a side below this run the small torch path (the kernels need 16-byte rows: multiples of 8 elements)
MIN_KERNEL_DIM = 8


class _Bucket:
    """Same-shape Muon matrices that are reduced, orthogonalised and pushed together.  `params` keeps every block's matrices
    adjacent, so the gradients of one block are a contiguous sub-range of the batch."""

    def __init__(self, rows: int, cols: int) -> None:
        self.rows, self.cols = rows, cols
        self.params: List[nn.Parameter] = []
        self.layers: List[int] = []
        self.packed: Optional[Tensor] = None      # [n, m, k] bf16 Polar Express input of the current step
        self.sumsq: Optional[Tensor] = None
        self.prepared: set = set()                # layers whose sub-range of `packed` is already filled this step

    def layer_range(self, layer: int) -> Tuple[int, int]:
        idx = [i for i, l in enumerate(self.layers) if l == layer]
        return (idx[0], idx[-1] + 1) if idx else (0, 0)


class FusedEngine:
    def __init__(self, model: nn.Module, training_config, optimizers: Dict[str, torch.optim.Optimizer],
                 dp_group=None, ep_size: int = 1, ep_group=None, expert_replica_group=None) -> None:
        self.model, self.cfg, self.optimizers = model, training_config, optimizers
        self.group = dp_group
        self.world, self.rank = du.world_size(dp_group), du.get_rank(dp_group)
        self.ep_size, self.ep_group = ep_size, ep_group
        self.device = next(model.parameters()).device
        wire = getattr(training_config, "grad_reduce_dtype", "fp32")
        if wire not in ("fp32", "bf16"):
            raise ValueError("grad_reduce_dtype must be 'fp32' or 'bf16'")
        self.wire_bf16 = wire == "bf16" and self.world > 1
        groups = model.optimizer_param_groups()
        named = dict(model.named_parameters())
        muon_names = [n for n, _ in groups["muon"]]
        expert_local = {n for n in muon_names if ".mlp.experts." in n} if ep_size > 1 else set()
        # ranks that hold the same experts as this one (itself included), in rank order
        self.replica_ranks = list(range(self.rank % ep_size, self.world, ep_size)) if ep_size > 1 else [self.rank]
        self.small = [(n, named[n]) for n in muon_names
                      if min(named[n].shape) < MIN_KERNEL_DIM or named[n].shape[1] % 8 or named[n].shape[0] % 8]
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
        self.grad_shadow = SymmetricBuffer(cursor, torch.bfloat16, self.device, dp_group) if self.wire_bf16 else None
        self.adamw_offsets: Dict[str, int] = {}
        cursor = 0
        for n, p in self.adamw_named:
            self.adamw_offsets[n] = cursor
            cursor += _aligned(p.numel())
        self.adamw_numel = _aligned(cursor, 4 * max(self.world, 1))
        self.adamw_param = SymmetricBuffer(self.adamw_numel, torch.float32, self.device, dp_group)
        self.adamw_grad = SymmetricBuffer(self.adamw_numel, torch.float32, self.device, dp_group)
        self.adamw_decay = torch.zeros(self.adamw_numel, dtype=torch.float32, device=self.device)
        self.barrier = PeerBarrier(self.device, dp_group)

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
        self.shared_buckets = self._make_buckets(self.owned_shared)
        self.local_buckets = self._make_buckets(self.owned_local)
        per = self.adamw_numel // self.world
        self.adamw_lo = self.rank * per
        self.adamw_n = per
        moment_dtype = optimizers["adamw"].moment_dtype
        self.adamw_m = torch.zeros(per, dtype=moment_dtype, device=self.device)
        self.adamw_v = torch.zeros(per, dtype=moment_dtype, device=self.device)
        self.adamw_step = 0
        self._import_optimizer_state()

        # ---- overlap of the gradient reduction with the backward pass -----------------------------------------------------
        # When the backward of a transformer block has been issued, this rank publishes a flag for that block; on a second
        # stream the owner of a matrix waits (bounded) for the block's flags of all ranks and then sums the block's gradients
        # out of the peers' buffers (with momentum and the bf16 pack) while the main stream continues with the earlier
        # blocks.  Orthogonalisation and the weight push stay behind the backward pass, where every bucket runs as one batch.
        wanted = getattr(training_config, "overlap_grad_reduce", None)
        self.overlap = bool(self.world > 1 and (self.world >= 4 if wanted is None else wanted))
        layers = sorted({l for b in self.shared_buckets for l in b.layers} | {self._layer_of(n) for n, _ in shared})
        self.layer_slot = {layer: i for i, layer in enumerate(layers)}
        self.layer_span: Dict[int, Tuple[int, int]] = {}      # element range of a block's matrices in the flat Muon buffers
        for n, p in shared:
            layer, off = self._layer_of(n), self.big_offsets[n]
            lo, hi = self.layer_span.get(layer, (off, off))
            self.layer_span[layer] = (min(lo, off), max(hi, off + _aligned(p.numel())))
        self.flags = SymmetricBuffer((len(layers) + 1) * max(self.world, 1), torch.int32, self.device, dp_group) if self.overlap else None
        self.step_word = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.overlap else None
        self._early_layers: set = set()
        # ---- CUDA graphs: forward + backward of one micro-step, captured per (input shape, window, loss scale) ----------------
        self.use_graphs = bool(getattr(training_config, "use_cuda_graphs", True) and self.device.type == "cuda")
        self._graphs: Dict[tuple, dict] = {}
        self._barrier()

    # ---- layout helpers ---------------------------------------------------------------------------------------------------
    @staticmethod
    def _layer_of(name: str) -> int:
        parts = name.split(".")
        return int(parts[2]) if len(parts) > 2 and parts[1] == "h" and parts[2].isdigit() else -1

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

    def _make_buckets(self, items: List[Tuple[str, nn.Parameter]]) -> List[_Bucket]:
        buckets: Dict[Tuple[int, int], _Bucket] = {}
        for n, p in sorted(items, key=lambda kv: self._layer_of(kv[0])):      # stable: a block's matrices stay adjacent
            rows, cols = p.shape
            if rows == 3 * cols:                      # fused (3d, d) projections are orthogonalised as three squares
                raise NotImplementedError("fused (3d, d) matrices are not laid out by this engine")
            b = buckets.setdefault((rows, cols), _Bucket(rows, cols))
            b.params.append(p)
            b.layers.append(self._layer_of(n))
        return list(buckets.values())

    def _barrier(self) -> None:
        self.barrier.sync()

    def set_comm_dry_run(self, enabled: bool) -> None:
        """Measurement mode: peer offsets collapse onto this rank and barriers are skipped (see `SymmetricBuffer.dry_run`)."""
        for buf in (self.grad_muon, self.compute, self.adamw_param, self.adamw_grad, self.grad_shadow, self.flags):
            if buf is not None:
                buf.dry_run = enabled
        self.barrier.dry_run = enabled

    def describe(self) -> Dict[str, object]:
        """What actually runs, for benchmark records."""
        return {"engine": type(self).__name__, "graphs": bool(self.use_graphs and self._graphs and any("graph" in e for e in self._graphs.values())),
                "grad_wire": "bf16" if self.wire_bf16 else "fp32", "overlap_grad_reduce": self.overlap}

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

    def drop_foreign_state(self) -> None:
        """After a resume every rank has loaded the whole Muon state; keep only the momentum of the matrices this rank updates,
        so that a stale copy of another owner's momentum can never be saved later."""
        muon = self.optimizers.get("muon")
        if muon is None:
            return
        mine = {id(p) for _, p in self.owned_shared + self.owned_local + self.small}
        for p in [p for p in muon.state if id(p) not in mine]:
            del muon.state[p]

    def contributes_state(self, name: str) -> bool:
        """Exactly one rank hands in a parameter's Muon state at save time: the owner of a shared matrix, the holder of an
        expert in the first expert-parallel group, rank 0 for the tiny matrices every rank updates."""
        if name in self.owners:
            return self.owners[name] == self.rank
        if self.ep_size > 1 and ".mlp.experts." in name:
            return self.rank < self.ep_size
        return self.rank == 0

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
        first-write / accumulate choice of the weight-gradient GEMMs is then fixed), no document ids, the plain chain of
        blocks (no activation checkpointing or offloading).  Cross-rank pieces are part of the graph: the overlapped gradient
        reduction (its flags take their value from a device word, the second stream forks from and joins the capturing
        stream) and the expert-parallel exchange (symmetric workspaces allocated during the eager warm-up steps, barriers
        whose epoch lives on the device, all sizes on the device)."""
        raw = self.model
        return (self.use_graphs and x.is_cuda and document_ids is None and self.cfg.grad_accum_mini_steps == 1
                and raw.training and torch.is_grad_enabled()
                and not getattr(raw, "use_activation_checkpointing", False) and getattr(raw, "activation_offloader", None) is None)

    def _run_forward_backward(self, model, x, y, document_ids, loss_scale: float, early: bool):
        """Forward + backward of one micro-step; with `early` the per-block hooks start the gradient reduction on the second
        stream, which is joined before this returns (so the sequence is one fork/join region: capturable)."""
        from ..ops import cuda_ops
        if early:
            cuda_ops.ext().bump_word(self.step_word)
            self._early_layers = set()
            for b in self.shared_buckets:
                b.prepared = set()
                n = len(b.params)
                m, k = min(b.rows, b.cols), max(b.rows, b.cols)
                b.packed = torch.empty((n, m, k), dtype=torch.bfloat16, device=self.device)
                b.sumsq = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.model.block_grad_hook = self._on_block_backward if early else None
        try:
            loss, token_loss, balance = model(x, y, document_ids=document_ids)
            (loss * loss_scale).backward()
        finally:
            self.model.block_grad_hook = None
        if early:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        return loss, token_loss, balance

    def _graphed_forward_backward(self, model, x, y, loss_scale: float, early: bool):
        """Third and later calls with the same key replay a captured graph of forward + backward (inputs are copied into the
        graph's static tensors; losses come back in static tensors); the first two run eagerly (they also warm every cache)."""
        from ..ops import cuda_ops
        window = getattr(getattr(self.model, "sliding_window_size", None), "host_value", None)
        key = (tuple(x.shape), tuple(y.shape), window, float(loss_scale), x.dtype, early)
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
                    loss, token_loss, balance = self._run_forward_backward(model, sx, sy, None, loss_scale, early)
            except Exception as exc:              # capture refused (an op that cannot be captured): stay eager from now on
                self.use_graphs = False
                self._graphs.clear()
                torch.cuda.synchronize()
                import sys
                print(f"CUDA graph capture of the training step failed ({type(exc).__name__}: {exc}); continuing without graphs",
                      file=sys.stderr)
                return None
            entry.update(graph=graph, x=sx, y=sy, outs=(loss.detach(), token_loss.detach(), balance.detach()),
                         launches=cuda_ops.launch_count() - before, early=set(self._early_layers),
                         packed=[(b.packed, b.sumsq, set(b.prepared)) for b in self.shared_buckets])
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
        if early:                                 # the replay filled the captured buffers: hand them to step()
            self._early_layers = set(entry["early"])
            for b, (packed, sumsq, prepared) in zip(self.shared_buckets, entry["packed"]):
                b.packed, b.sumsq, b.prepared = packed, sumsq, set(prepared)
        return entry["outs"]

    def forward_backward(self, model, x, y, document_ids, loss_scale: float, last_micro_step: bool):
        from ..ops import cuda_ops
        cuda_ops.set_loss_scale(loss_scale)
        early = self.overlap and last_micro_step and self.optimizers.get("muon") is not None and not self.barrier.dry_run
        if self._graph_eligible(model, x, document_ids):
            outs = self._graphed_forward_backward(model, x, y, loss_scale, early)
            if outs is not None:
                return outs
        return self._run_forward_backward(model, x, y, document_ids, loss_scale, early)

    def _prepare(self, b: _Bucket, lo: int, hi: int, deltas_grad: List[int]) -> None:
        """Reduce + momentum + Nesterov + bf16 pack for matrices [lo, hi) of a bucket into its `packed` / `sumsq`."""
        from ..ops import cuda_ops
        if hi <= lo:
            return
        c = cuda_ops.ext()
        muon = self.optimizers["muon"]
        g = muon.param_groups[0]
        batch = b.params[lo:hi]
        bufs = []
        for p in batch:
            state = muon.state[p]
            if "momentum_buffer" not in state:
                state["momentum_buffer"] = torch.zeros_like(p.data)
            bufs.append(state["momentum_buffer"])
        wire = self.wire_bf16 and len(deltas_grad) > 1
        c.rs_muon_prepare(cuda_ops._ptr_table([p.main_grad for p in batch]), cuda_ops._ptr_table(bufs), b.packed[lo:hi], b.sumsq[lo:hi],
                          b.rows, b.cols, b.cols, b.cols, g["momentum"], g["nesterov"], b.rows > b.cols, deltas_grad, normalize=False,
                          grad_base=self.grad_muon.tensor if wire else None, shadow=self.grad_shadow.tensor if wire else None)

    def _on_block_backward(self, layer: int) -> None:
        """Called from the backward pass once every gradient of block `layer` has been issued on the current stream."""
        from ..ops import cuda_ops
        c = cuda_ops.ext()
        if layer in self._early_layers or layer not in self.layer_slot:
            return
        self._early_layers.add(layer)
        if self.wire_bf16:                        # the bf16 shadow of this block's gradients, which the peers will read
            lo, hi = self.layer_span[layer]
            c.cast_bf16(self.grad_muon.tensor[lo:hi], self.grad_shadow.tensor[lo:hi])
        slot = self.layer_slot[layer]
        c.flag_signal(self.flags.tensor, self.flags.deltas, slot * self.world + self.rank, 0, self.step_word)
        work = [(b,) + b.layer_range(layer) for b in self.shared_buckets]
        work = [(b, lo, hi) for b, lo, hi in work if hi > lo]
        if not work:
            return
        ready = torch.cuda.Event()
        ready.record()
        deltas = (self.grad_shadow if self.wire_bf16 else self.grad_muon).deltas
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ready)
            c.flag_wait(self.flags.tensor, slot * self.world, self.world, 0, self.step_word)
            for b, lo, hi in work:
                self._prepare(b, lo, hi, deltas)
                b.prepared.add(layer)

    def _muon_update(self, buckets: List[_Bucket], deltas_grad: List[int], deltas_compute: List[int], lr: float) -> None:
        """Whatever of a bucket is not prepared yet is reduced now; then Polar Express and the push run on the whole bucket."""
        from ..ops import cuda_ops
        c = cuda_ops.ext()
        for b in buckets:
            n = len(b.params)
            if n == 0:
                continue
            m, k = min(b.rows, b.cols), max(b.rows, b.cols)
            if b.packed is None:
                b.packed = torch.empty((n, m, k), dtype=torch.bfloat16, device=self.device)
                b.sumsq = torch.zeros(n, dtype=torch.float32, device=self.device)
            # maximal runs of matrices whose layer has not been prepared beside the backward pass
            start = None
            for i in range(n + 1):
                pending = i < n and b.layers[i] not in b.prepared
                if pending and start is None:
                    start = i
                elif not pending and start is not None:
                    self._prepare(b, start, i, deltas_grad)
                    start = None
            update = cuda_ops.polar_express_bf16(b.packed, b.sumsq)      # the first iteration's epilogues apply the normalisation
            alpha = -lr * max(b.rows, b.cols) ** 0.5
            c.muon_apply_push(cuda_ops._ptr_table([p.data for p in b.params]), cuda_ops._ptr_table([p.compute for p in b.params]),
                              update, b.rows, b.cols, b.cols, b.cols, alpha, b.rows > b.cols, deltas_compute)
            b.packed = b.sumsq = None
            b.prepared = set()

    def step(self) -> None:
        from ..ops import cuda_ops
        from ..ops import reference as ref
        c = cuda_ops.ext()
        muon, adamw = self.optimizers.get("muon"), self.optimizers["adamw"]
        # a matrix whose GEMM ran outside the kernels (a shape they do not cover, e.g. a router with fewer than 8 experts goes
        # through torch) has its gradient in `.grad`: move it into the flat buffer, where the reduction looks for it
        for _, p in self.big + self.small:
            if p.grad is not None:
                if p.grad_ready:
                    p.main_grad.add_(p.grad)
                else:
                    p.main_grad.copy_(p.grad)
                    p.grad_ready = True
                p.grad = None
        if self.wire_bf16 and muon is not None:
            # peers read a bf16 shadow of the gradients; blocks handled beside the backward pass were cast there
            todo = [self.layer_span[l] for l in self.layer_span if l not in self._early_layers]
            if len(todo) == len(self.layer_span):
                n = self.grad_muon.tensor.numel()
                c.cast_bf16(self.grad_muon.tensor[:n], self.grad_shadow.tensor[:n])
            else:
                for lo, hi in todo:
                    c.cast_bf16(self.grad_muon.tensor[lo:hi], self.grad_shadow.tensor[lo:hi])
                if self.replica_ranks != [self.rank] and self.owned_local:
                    n = self.grad_muon.tensor.numel()
                    c.cast_bf16(self.grad_muon.tensor[:n], self.grad_shadow.tensor[:n])
        self._barrier()                                   # every rank's gradients are complete
        if muon is not None:
            g = muon.param_groups[0]
            lr, momentum, nesterov = g["lr"], g["momentum"], g["nesterov"]
            if g["backend"] != "polarexpress":
                raise NotImplementedError("the fused engine implements the Polar Express backend")
            grad_src = self.grad_shadow if self.wire_bf16 else self.grad_muon
            self._early_layers = set()
            self._muon_update(self.shared_buckets, grad_src.deltas, self.compute.deltas, lr)
            # experts under expert parallelism: summed over the ranks that hold the same experts (none when every rank holds
            # different ones), updated by every holder identically, stored locally
            replica_deltas = [grad_src.deltas[r] for r in self.replica_ranks] if len(self.replica_ranks) > 1 else [0]
            self._muon_update(self.local_buckets, replica_deltas, [0], lr)
            # matrices too narrow for the kernels (rows or columns not a multiple of 8): every rank averages them out of all
            # buffers and repeats the small update with torch ops
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
        """Optimizer state in the unsharded torch layout (per-parameter `momentum_buffer`; `step`, `exp_avg`, `exp_avg_sq`),
        keyed by the unsharded model's parameter order.  Collective."""
        from ..checkpointing.checkpoint import merge_optimizer_state
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
            out["muon"] = merge_optimizer_state(self.model, self.optimizers["muon"], self.contributes_state, self.group)
        return out


def build_cuda_engine(model, training_config, optimizers, ep_size: int = 1, ep_group=None, expert_replica_group=None):
    """The fused engine when it is requested (`use_fused_collectives`) and the model fits its assumptions (fp32 masters, Polar
    Express Muon, no fused (3d, d) projections); otherwise the NCCL engine.  A failure to set the fused engine up (symmetric
    memory unavailable) raises, unless `allow_nccl_fallback` asks for the NCCL engine in that case."""
    usable = (training_config.use_fused_collectives and "muon" in optimizers
              and optimizers["muon"].param_groups[0]["backend"] == "polarexpress"
              and all(p.dtype == torch.float32 for p in model.parameters())
              and not any(p.shape[0] == 3 * p.shape[1] for p in model.parameters() if p.dim() == 2))
    if usable:
        try:
            return FusedEngine(model, training_config, optimizers, dp_group=None, ep_size=ep_size, ep_group=ep_group,
                               expert_replica_group=expert_replica_group)
        except Exception as exc:
            if not getattr(training_config, "allow_nccl_fallback", False):
                raise
            if du.get_rank() == 0:
                import sys
                print(f"fused engine unavailable ({type(exc).__name__}: {exc}); using NCCL collectives", file=sys.stderr)
    return CudaHostEngine(model, training_config, optimizers, dp_group=None, ep_size=ep_size, expert_replica_group=expert_replica_group)
