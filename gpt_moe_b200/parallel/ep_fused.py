"""Expert parallelism with dispatch and combine fused into the all-to-all (CUDA, peer memory over NVLink).

Every rank of the expert-parallel group maps the other ranks' receive / return buffers (symmetric memory).  The
forward of one MoE layer is then

    route locally -> store my per-expert counts into every rank's count table          | barrier
    plan (every rank derives the owners' padded layouts from the full table)
    dispatch: each (token, slot) row is STORED into the owner's receive buffer at its final row   | barrier
    grouped up GEMM -> activation -> grouped down GEMM on the local experts (tcgen05 kernels)   | barrier
    combine: each token LOADS its slots' rows from the owners' return buffers and applies the gates

and the backward runs the same two kernels the other way round (dispatch of gate * dOut with the gate gradient's dot
product in the same pass; combine of the input gradients with unit gates).  No row is staged, sorted or copied for the
exchange, and there are no host synchronisations: sizes stay on the device.  Buffers hold the worst case by default
(every slot of every rank routed to one rank); `ep_capacity_factor > 0` shrinks them to that many times a rank's own
slots, and a row that then does not fit sets the device status word, which invalidates the step instead of dropping
tokens silently.

The NCCL path (`parallel.ep.expert_parallel_moe`) is the baseline this replaces and the oracle of the tests.
The reference keeps all experts on every rank (model/feedforward/moe.py:30); expert parallelism is an addition.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
from torch import Tensor

from ..ops import cuda_ops as co
from . import dist_utils as du

BF16 = torch.bfloat16


class EPWorkspace:
    """Symmetric buffers of one expert-parallel group: count table, one return buffer, one gradient receive buffer, and one
    receive buffer per MoE layer (it doubles as the saved grouped-GEMM input of that layer, so nothing is copied)."""

    def __init__(self, group, slots: int, d: int, experts: int, device, capacity_factor: float = 0.0) -> None:
        from .fused_engine import PeerBarrier, SymmetricBuffer
        self.group = group
        self.world, self.rank = du.world_size(group), du.get_rank(group)
        assert experts % self.world == 0
        self.experts, self.per_rank, self.d, self.slots = experts, experts // self.world, d, slots
        # capacity_factor <= 0: room for the worst case (every slot of every rank routed to this rank's experts)
        rows = self.world * slots if capacity_factor <= 0 else min(self.world * slots, int(capacity_factor * slots + 0.5))
        self.cap_rows = (rows + 255) // 256 * 256 + self.per_rank * 256
        self.device = device
        self._make = lambda numel, dtype: SymmetricBuffer(numel, dtype, device, group)
        self.table = self._make(self.world * experts, torch.int32)
        self.ret = self._make(self.cap_rows * d, BF16)
        self.grad_recv = self._make(self.cap_rows * d, BF16)
        self.layer_recv: Dict[int, object] = {}
        self._barrier = PeerBarrier(device, group)

    def recv_for(self, layer_key: int):
        buf = self.layer_recv.get(layer_key)
        if buf is None:
            buf = self.layer_recv[layer_key] = self._make(self.cap_rows * self.d, BF16)
        return buf

    def rows(self, buf) -> Tensor:
        return buf.tensor[: self.cap_rows * self.d].view(self.cap_rows, self.d)

    def barrier(self) -> None:
        """Bounded device-side barrier of the expert-parallel group (status 601 if a peer never arrives)."""
        self._barrier.sync()


_workspaces: Dict[tuple, EPWorkspace] = {}


def workspace_for(group, slots: int, d: int, experts: int, device, capacity_factor: float) -> EPWorkspace:
    key = (id(group), slots, d, experts, str(device), capacity_factor)
    ws = _workspaces.get(key)
    if ws is None:
        ws = _workspaces[key] = EPWorkspace(group, slots, d, experts, device, capacity_factor)
    return ws


def release_workspaces() -> None:
    _workspaces.clear()


class _FusedEPMoEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden: Tensor, gates: Tensor, top_idx: Tensor, activation: str, ws: EPWorkspace, layer_key: int, mx: bool,
                *weights: Tensor):
        """`mx`: the expert projections are MXFP8 — forward and input-gradient grouped GEMMs read e4m3 operands (received rows and
        received gradients are quantised where they land, activations by the kernel that writes them); weight gradients stay
        bf16 x bf16 -> fp32."""
        c = co.ext()
        n_local = ws.per_rank
        up, down = weights[:n_local], weights[n_local:]
        h2 = co._as_bf16_2d(hidden)
        idx = top_idx.contiguous()
        gates32 = gates.detach().float().contiguous()
        dest, _src, local_seg_ends, counts, _tiles, _meta = c.route(idx, ws.experts)
        c.ep_push_counts(counts, ws.table.tensor, ws.table.deltas, ws.rank)
        ws.barrier()
        my_base, seg_ends, valid_ends, tile_expert, meta = c.ep_plan(ws.table.tensor, ws.world, ws.rank, ws.experts, ws.cap_rows)
        recv_buf = ws.recv_for(layer_key)
        packed = ws.rows(recv_buf)
        c.ep_zero_pads(packed, seg_ends, valid_ends)
        (route_row,) = c.ep_dispatch(h2, idx, dest, local_seg_ends, my_base, None, None, packed, recv_buf.deltas, n_local)
        ws.barrier()
        y = ws.rows(ws.ret)
        if mx:
            from ..ops import mxfp8
            w_up, uq, usf, uqt, usft = mxfp8._quantized_weight(up, stack=True)
            w_down, dq, dsf, dqt, dsft = mxfp8._quantized_weight(down, stack=True)
            pq, psf = c.mxfp8_quantize(packed, meta[1:2])
            pre = torch.empty((ws.cap_rows, w_up.shape[1]), dtype=BF16, device=hidden.device)
            c.gemm_mxfp8(pq, psf, uq, usf, pre, 1.0, tile_expert, meta)
            act, aq, asf = c.activation_fwd(pre, activation, meta, quantize=True)
            c.gemm_mxfp8(aq, asf, dq, dsf, y, 1.0, tile_expert, meta)
            w_up, w_down = (uqt, usft), (dqt, dsft)            # what the backward needs of the weights
        else:
            w_up, w_down = co.stacked_weight(up), co.stacked_weight(down)
            pre = torch.empty((ws.cap_rows, w_up.shape[1]), dtype=BF16, device=hidden.device)
            c.gemm_bf16(packed, w_up, pre, False, False, 1.0, 0.0, None, False, 1, tile_expert, meta, None)
            (act,) = c.activation_fwd(pre, activation, meta)
            c.gemm_bf16(act, w_down, y, False, False, 1.0, 0.0, None, False, 1, tile_expert, meta, None)
            w_up, w_down = (w_up,), (w_down,)
        ws.barrier()
        out, y_rows = c.ep_combine(y, idx, route_row, gates32, True, ws.ret.deltas, n_local)
        ctx.save_for_backward(packed, pre, act, y_rows, idx, dest, local_seg_ends, my_base, route_row, seg_ends, valid_ends, tile_expert, meta,
                              gates32, *w_up, *w_down)
        ctx.activation, ctx.ws, ctx.weights, ctx.mx = activation, ws, weights, mx
        ctx.hidden_meta = (hidden.shape, hidden.dtype, gates.dtype)
        ctx.mark_non_differentiable(top_idx)
        return out.view(*hidden.shape[:-1], out.shape[-1]).to(hidden.dtype)

    @staticmethod
    def backward(ctx, dout: Tensor):
        c = co.ext()
        (packed, pre, act, y_rows, idx, dest, local_seg_ends, my_base, route_row, seg_ends, valid_ends, tile_expert, meta,
         gates32) = ctx.saved_tensors[:14]
        saved_w = ctx.saved_tensors[14:]
        mx = ctx.mx
        ws: EPWorkspace = ctx.ws
        e = ws.per_rank
        up, down = ctx.weights[:e], ctx.weights[e:]
        shape, dtype, gdtype = ctx.hidden_meta
        d2 = co._as_bf16_2d(dout)
        dy = ws.rows(ws.grad_recv)
        c.ep_zero_pads(dy, seg_ends, valid_ends)
        _, dgates = c.ep_dispatch(d2, idx, dest, local_seg_ends, my_base, gates32, y_rows, dy, ws.grad_recv.deltas, e)
        ws.barrier()
        dact = torch.empty_like(act)
        if mx:
            uqt, usft, dqt, dsft = saved_w
            gq, gsf = c.mxfp8_quantize(dy, meta[1:2])
            c.gemm_mxfp8(gq, gsf, dqt, dsft, dact, 1.0, tile_expert, meta)
        else:
            w_up, w_down = saved_w
            c.gemm_bf16(dy, w_down, dact, False, True, 1.0, 0.0, None, False, 1, tile_expert, meta, None)
        grads: List[Optional[Tensor]] = [None] * (2 * e)
        ends = seg_ends

        def wgrad(a: Tensor, b: Tensor, params: Sequence[Tensor], offset: int) -> None:
            target = co._grad_targets(params)
            if target is not None:
                c.gemm_bf16(a, b, target.view(e, params[0].shape[0], params[0].shape[1]), True, True, 1.0, 0.0, None,
                            co._take_accumulate_flag(params), 2, None, None, ends)
                return
            dw = torch.empty((e, params[0].shape[0], params[0].shape[1]), dtype=torch.float32, device=a.device)
            c.gemm_bf16(a, b, dw, True, True, 1.0, 0.0, None, False, 2, None, None, ends)
            for i, p in enumerate(params):
                grads[offset + i] = dw[i].to(p.dtype)

        wgrad(dy, act, down, e)
        res = c.activation_bwd(dact, pre, ctx.activation, meta, quantize=mx)
        dpre = res[0]
        wgrad(dpre, packed, up, 0)
        dpacked = ws.rows(ws.ret)
        if mx:
            c.gemm_mxfp8(res[1], res[2], uqt, usft, dpacked, 1.0, tile_expert, meta)
        else:
            c.gemm_bf16(dpre, w_up, dpacked, False, True, 1.0, 0.0, None, False, 1, tile_expert, meta, None)
        ws.barrier()
        (dhidden,) = c.ep_combine(dpacked, idx, route_row, None, False, ws.ret.deltas, e)
        return (dhidden.view(shape).to(dtype), dgates.to(gdtype), None, None, None, None, None) + tuple(grads)


def fused_expert_parallel_moe(moe, hidden: Tensor, top_idx: Tensor, gates: Tensor, args: dict) -> Tensor:
    """Drop-in for `parallel.ep.expert_parallel_moe` on CUDA (bf16 experts without biases)."""
    if args["up_biases"] is not None or args["down_biases"] is not None:
        raise NotImplementedError("expert biases are not supported by the fused expert-parallel path")
    h2 = hidden.reshape(-1, hidden.shape[-1])
    ws = workspace_for(moe.ep_group, top_idx.numel(), h2.shape[-1], moe.num_experts, hidden.device, float(getattr(moe, "ep_capacity_factor", 0.0)))
    up, down = args["up_weights"], args["down_weights"]
    wants_mx = args.get("up_precision") in ("mxfp8", "fp8") or args.get("down_precision") in ("mxfp8", "fp8")
    mx = bool(wants_mx and up[0].shape[1] % 128 == 0 and up[0].shape[0] % 128 == 0 and down[0].shape[1] % 128 == 0 and down[0].shape[0] % 128 == 0)
    return _FusedEPMoEFn.apply(h2, gates, top_idx, args["activation"], ws, id(moe), mx, *up, *down)


def supported(moe, hidden: Tensor) -> bool:
    d = hidden.shape[-1]
    return bool(hidden.is_cuda and getattr(moe, "ep_fused", False) and d % 8 == 0 and moe.num_experts <= 128 and moe.ep_size <= 16)
