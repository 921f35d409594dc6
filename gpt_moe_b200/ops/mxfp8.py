"""MXFP8 linear layers on the block-scaled tensor-core path.

Forward and input-gradient GEMMs run on e4m3 operands with one UE8M0 scale per 32 elements of the contraction
dimension (`tcgen05.mma kind::mxf8f6f4.block_scale`); the weight-gradient GEMM stays in bf16 with fp32
accumulation straight into the optimizer's gradient buffer, so the optimizer sees the same gradient layout
as in the bf16 path.  Quantised weights (row-major for forward, transposed for the input gradient) are cached
until the parameters change.  The oracle is `ops.reference.mxfp8_linear`.

Reference counterparts: model/linear/fp8/custom/dense.py:124-167 (quantise, DeepGEMM forward, bf16 backward) and
model/linear/fp8/custom/grouped.py:228-330 (grouped experts); the reference scales 128-element blocks in software,
here the 32-element MX format is applied by the MMA itself.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
from torch import Tensor

from . import cuda_ops as co

BF16 = torch.bfloat16


def _quantized_weight(weights: Sequence[Tensor], stack: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """(bf16 weight, e4m3 bytes, scales, transposed e4m3 bytes, transposed scales) of cat / stack of `weights`."""
    w = co.stacked_weight(weights) if stack else co.bf16_weight(weights)

    def build(_old):
        c = co.ext()
        wc = w if w.is_contiguous() else w.contiguous()
        q, sf = c.mxfp8_quantize(wc)
        qt, sft = c.mxfp8_quantize_transposed(wc)
        return q, sf, qt, sft

    q, sf, qt, sft = co._cached(("mxfp8", stack) + tuple(id(p) for p in weights), weights, build)
    return w, q, sf, qt, sft


def supported(k: int, n: int) -> bool:
    return k % 128 == 0 and n % 128 == 0


class _MXFP8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, n_weights: int, *weights: Tensor) -> Tensor:
        c = co.ext()
        x2 = co._as_bf16_2d(x)
        w, wq, wsf, wqt, wsft = _quantized_weight(weights, stack=False)
        xq, xsf = c.mxfp8_quantize(x2)
        y = torch.empty((x2.shape[0], w.shape[0]), dtype=BF16, device=x.device)
        c.gemm_mxfp8(xq, xsf, wq, wsf, y)
        ctx.save_for_backward(x2, wqt, wsft)
        ctx.weights = weights
        ctx.x_shape, ctx.x_dtype, ctx.w_shape = x.shape, x.dtype, tuple(w.shape)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy: Tensor):
        c = co.ext()
        x2, wqt, wsft = ctx.saved_tensors
        weights = ctx.weights
        dy2 = co._as_bf16_2d(dy)
        dx = None
        if ctx.needs_input_grad[0]:
            gq, gsf = c.mxfp8_quantize(dy2)
            dx = torch.empty_like(x2)
            c.gemm_mxfp8(gq, gsf, wqt, wsft, dx)                       # dX = Q(dY) Q(W^T)^T, blocks along N
            dx = dx.view(ctx.x_shape).to(ctx.x_dtype)
        grads: List[Optional[Tensor]] = [None] * len(weights)
        if any(ctx.needs_input_grad[2:]):
            target = co._grad_targets(weights)
            if target is not None:
                c.gemm_bf16(dy2, x2, target, True, True, 1.0, 0.0, None, co._take_accumulate_flag(weights))
            else:
                dw = torch.empty(ctx.w_shape, dtype=torch.float32, device=x2.device)
                c.gemm_bf16(dy2, x2, dw, True, True)
                r = 0
                for i, p in enumerate(weights):
                    grads[i] = dw[r: r + p.shape[0]].to(p.dtype)
                    r += p.shape[0]
        return (dx, None) + tuple(grads)


def mxfp8_linear_multi(x: Tensor, weights: Sequence[Tensor]) -> Tensor:
    k = weights[0].shape[1]
    n = sum(w.shape[0] for w in weights)
    if not supported(k, n):
        return co._LinearFn.apply(x, len(weights), *weights)
    return _MXFP8LinearFn.apply(x, len(weights), *weights)


class _MXFP8MoEExpertsFn(torch.autograd.Function):
    """Same data flow as the bf16 expert function; the four grouped forward / input-gradient GEMMs read e4m3."""

    @staticmethod
    def forward(ctx, hidden: Tensor, gates: Tensor, top_idx: Tensor, activation: str, num_experts: int, *weights: Tensor):
        c = co.ext()
        up, down = weights[:num_experts], weights[num_experts:]
        top_k = top_idx.shape[1]
        h2 = co._as_bf16_2d(hidden)
        gates32 = gates.detach().float().contiguous()
        dest, src_of_row, seg_ends, counts, tile_expert, meta = c.route(top_idx.contiguous(), num_experts)
        packed = c.gather_rows(h2, src_of_row, meta, top_k)
        w_up, uq, usf, uqt, usft = _quantized_weight(up, stack=True)
        w_down, dq, dsf, dqt, dsft = _quantized_weight(down, stack=True)
        rows = meta[1:2]
        cap = packed.shape[0]
        pq, psf = c.mxfp8_quantize(packed, rows)
        pre = torch.empty((cap, w_up.shape[1]), dtype=BF16, device=hidden.device)
        c.gemm_mxfp8(pq, psf, uq, usf, pre, 1.0, tile_expert, meta)
        act = c.activation_fwd(pre, activation, meta)
        aq, asf = c.mxfp8_quantize(act, rows)
        y = torch.empty((cap, w_down.shape[1]), dtype=BF16, device=hidden.device)
        c.gemm_mxfp8(aq, asf, dq, dsf, y, 1.0, tile_expert, meta)
        out = c.combine_fwd(y, dest, gates32)
        ctx.save_for_backward(packed, pre, act, y, dest, src_of_row, seg_ends, tile_expert, meta, gates32, uqt, usft, dqt, dsft)
        ctx.activation, ctx.num_experts, ctx.weights = activation, num_experts, weights
        ctx.hidden_meta = (hidden.shape, hidden.dtype, gates.dtype)
        ctx.mark_non_differentiable(top_idx)
        return out.view(*hidden.shape[:-1], out.shape[-1]).to(hidden.dtype)

    @staticmethod
    def backward(ctx, dout: Tensor):
        c = co.ext()
        packed, pre, act, y, dest, src_of_row, seg_ends, tile_expert, meta, gates32, uqt, usft, dqt, dsft = ctx.saved_tensors
        e = ctx.num_experts
        up, down = ctx.weights[:e], ctx.weights[e:]
        shape, dtype, gdtype = ctx.hidden_meta
        rows = meta[1:2]
        d2 = co._as_bf16_2d(dout)
        dy, dgates = c.combine_bwd(d2, y, src_of_row, gates32, meta)
        gq, gsf = c.mxfp8_quantize(dy, rows)
        dact = torch.empty_like(act)
        c.gemm_mxfp8(gq, gsf, dqt, dsft, dact, 1.0, tile_expert, meta)
        grads: List[Optional[Tensor]] = [None] * (2 * e)

        def wgrad(a: Tensor, b: Tensor, params: Sequence[Tensor], offset: int) -> None:
            target = co._grad_targets(params)
            if target is not None:
                c.gemm_bf16(a, b, target.view(e, params[0].shape[0], params[0].shape[1]), True, True, 1.0, 0.0, None,
                            co._take_accumulate_flag(params), 2, None, None, seg_ends)
                return
            dw = torch.empty((e, params[0].shape[0], params[0].shape[1]), dtype=torch.float32, device=a.device)
            c.gemm_bf16(a, b, dw, True, True, 1.0, 0.0, None, False, 2, None, None, seg_ends)
            for i, p in enumerate(params):
                grads[offset + i] = dw[i].to(p.dtype)

        wgrad(dy, act, down, e)
        dpre = c.activation_bwd(dact, pre, ctx.activation, meta)
        wgrad(dpre, packed, up, 0)
        dhidden = None
        if ctx.needs_input_grad[0]:
            pq, psf = c.mxfp8_quantize(dpre, rows)
            dpacked = torch.empty_like(packed)
            c.gemm_mxfp8(pq, psf, uqt, usft, dpacked, 1.0, tile_expert, meta)
            dhidden = c.combine_fwd(dpacked, dest, torch.ones_like(gates32)).view(shape).to(dtype)
        return (dhidden, dgates.to(gdtype), None, None, None) + tuple(grads)


def mxfp8_moe_experts(hidden, top_idx, gates, up_weights, down_weights, activation):
    d, h_up = up_weights[0].shape[1], up_weights[0].shape[0]
    h_down = down_weights[0].shape[1]
    if not (supported(d, h_up) and supported(h_down, down_weights[0].shape[0])):
        return co._MoEExpertsFn.apply(hidden, gates, top_idx, activation, len(up_weights), *up_weights, *down_weights)
    return _MXFP8MoEExpertsFn.apply(hidden, gates, top_idx, activation, len(up_weights), *up_weights, *down_weights)
