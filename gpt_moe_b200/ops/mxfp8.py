"""MXFP8 linear layers on the block-scaled tensor-core path.

Forward and input-gradient GEMMs run on e4m3 operands with one UE8M0 scale per 32 elements of the contraction
dimension (`tcgen05.mma kind::mxf8f6f4.block_scale`, CTA pairs on 256 x 256 tiles); the weight-gradient GEMM stays in
bf16 with fp32 accumulation straight into the optimizer's gradient buffer, so the optimizer sees the same gradient
layout as in the bf16 path.

Nothing on the hot path runs a quantisation pass of its own.  The kernel that PRODUCES a GEMM operand writes its e4m3
payload and scale records next to the bf16 tensor (which the bf16 weight-gradient GEMM still reads):
  RMSNorm (+ residual)        -> input of the QKV projection            (`rmsnorm_fwd(quantize=True)`)
  expert gather               -> input of the up projection             (`gather_rows(quantize=True)`)
  activation forward          -> input of the down projection           (`activation_fwd(quantize=True)`)
  gated-combine backward      -> dY of the down projection              (`combine_bwd(quantize=True)`)
  activation backward         -> dY of the up projection                (`activation_bwd(quantize=True)`)
  RoPE / QK-norm backward     -> dY of the QKV projection               (`rope_qknorm_bwd(quantize=True)`)
  attention forward epilogue  -> input of the output projection         (`attn_fwd(quantize=True)`)
Only the output projection's dY is quantised by `mxfp8_quantize`, one pass over a [tokens, hidden] matrix.  Quantised weights — row-wise for the forward GEMM and
transposed for the input-gradient GEMM, both from one pass over the bf16 weight — are cached until the parameters change.
The oracle is `ops.reference.mxfp8_linear` / `mxfp8_quantize`.

Reference counterparts: model/linear/fp8/custom/dense.py:124-167 (quantise, DeepGEMM forward, backward),
model/linear/fp8/custom/rms_norm.py:23-55, model/linear/fp8/custom/grouped.py:15-84 and :228-330 (producers that quantise
while they gather / activate), model/attention/qkv_norm_rope_fp8.py:95-226 (backward that re-quantises dQ/dK/dV); the
reference scales 128-element blocks in software, here the 32-element MX format is applied by the MMA itself.
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
        wc = w if w.is_contiguous() else w.contiguous()
        return tuple(co.ext().mxfp8_quantize_weight(wc))

    q, sf, qt, sft = co._cached(("mxfp8", stack) + tuple(id(p) for p in weights), weights, build)
    return w, q, sf, qt, sft


def supported(k: int, n: int) -> bool:
    return k % 128 == 0 and n % 128 == 0


def clear_quantized_weights() -> None:
    """Forget every cached quantised weight (they are rebuilt on next use)."""
    for key in [k for k in co._weight_cache if isinstance(k, tuple) and k and k[0] == "mxfp8"]:
        del co._weight_cache[key]


def prepare_block_weights(block) -> None:
    """Fill the quantised-weight cache for the MXFP8 projections of one transformer block."""
    attn = getattr(block, "attn", None)
    if attn is not None and hasattr(attn, "q_proj") and hasattr(attn, "k_proj") and attn.q_proj.precision in ("mxfp8", "fp8"):
        ws = (attn.q_proj.weight, attn.k_proj.weight, attn.v_proj.weight)
        if supported(ws[0].shape[1], sum(w.shape[0] for w in ws)):
            _quantized_weight(ws, stack=False)
    if attn is not None and hasattr(attn, "out_proj") and attn.out_proj.precision in ("mxfp8", "fp8"):
        w = attn.out_proj.weight
        if supported(w.shape[1], w.shape[0]):
            _quantized_weight((w,), stack=False)
    mlp = getattr(block, "mlp", None)
    if mlp is not None and hasattr(mlp, "local_experts"):
        experts = mlp.local_experts()
        if experts and experts[0].up_proj.precision in ("mxfp8", "fp8"):
            ups, downs = [m.up_proj.weight for m in experts], [m.down_proj.weight for m in experts]
            if supported(ups[0].shape[1], ups[0].shape[0]) and supported(downs[0].shape[1], downs[0].shape[0]):
                _quantized_weight(ups, stack=True)
                _quantized_weight(downs, stack=True)


def _weight_grads(c, dy2: Tensor, x2: Tensor, weights: Sequence[Tensor], w_shape, needs: Sequence[bool]) -> List[Optional[Tensor]]:
    """bf16 x bf16 -> fp32 weight gradient of cat(weights): into the flat gradient buffer when the engine provides one."""
    grads: List[Optional[Tensor]] = [None] * len(weights)
    if not any(needs):
        return grads
    target = co._grad_targets(weights)
    if target is not None:
        c.gemm_bf16(dy2, x2, target, True, True, 1.0, 0.0, None, co._take_accumulate_flag(weights))
        return grads
    dw = torch.empty(w_shape, dtype=torch.float32, device=x2.device)
    c.gemm_bf16(dy2, x2, dw, True, True)
    r = 0
    for i, p in enumerate(weights):
        grads[i] = dw[r: r + p.shape[0]].to(p.dtype)
        r += p.shape[0]
    return grads


def _attached_copy(x: Tensor) -> Tuple[Optional[Tensor], Optional[Tensor]]:
    """The MXFP8 copy its producer attached to a GEMM input (`x.mxq`, see `cuda_ops.residual_rms_norm`), if any."""
    attached = getattr(x, "mxq", None)
    rows = x.numel() // x.shape[-1]
    if attached is not None and tuple(attached[0].shape) == (rows, x.shape[-1]):
        return attached
    return None, None


class _MXFP8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, xq: Optional[Tensor], xsf: Optional[Tensor], *weights: Tensor) -> Tensor:
        c = co.ext()
        x2 = co._as_bf16_2d(x)
        w, wq, wsf, wqt, wsft = _quantized_weight(weights, stack=False)
        if xq is None:
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
        grads = _weight_grads(c, dy2, x2, weights, ctx.w_shape, ctx.needs_input_grad[3:])
        return (dx, None, None) + tuple(grads)


def mxfp8_linear_multi(x: Tensor, weights: Sequence[Tensor]) -> Tensor:
    k = weights[0].shape[1]
    n = sum(w.shape[0] for w in weights)
    if not supported(k, n):
        return co._LinearFn.apply(x, len(weights), *weights)
    xq, xsf = _attached_copy(x)
    return _MXFP8LinearFn.apply(x, xq, xsf, *weights)


class _MXFP8QKVAttentionFn(torch.autograd.Function):
    """QKV projection (MXFP8) -> RoPE + QK-norm -> causal / sliding-window attention as one autograd node.  Backward: attention
    backward -> RoPE / QK-norm backward, which also emits the MXFP8 copy of the packed dQKV rows -> input-gradient GEMM on
    that copy, weight-gradient GEMM (bf16) on the bf16 rows.  The packed gradient is never read by a quantisation pass."""

    @staticmethod
    def forward(ctx, x: Tensor, xq: Optional[Tensor], xsf: Optional[Tensor], cos, sin, q_scale, k_scale, cfg: tuple, doc_start,
                *weights: Tensor):
        c = co.ext()
        batch, seq_len, hq, hk, d, eps, rms, smin, smax, window, scale, softcap, quant_out = cfg
        x2 = co._as_bf16_2d(x)
        w, wq, wsf, wqt, wsft = _quantized_weight(weights, stack=False)
        if xq is None:
            xq, xsf = c.mxfp8_quantize(x2)
        qkv = torch.empty((x2.shape[0], w.shape[0]), dtype=BF16, device=x.device)
        c.gemm_mxfp8(xq, xsf, wq, wsf, qkv)
        out = torch.empty_like(qkv)
        qs = None if q_scale is None else q_scale.detach().float().reshape(-1).contiguous()
        ks = None if k_scale is None else k_scale.detach().float().reshape(-1).contiguous()
        c.rope_qknorm_fwd(qkv, out, cos, sin, qs, ks, seq_len, hq, hk, d, eps, rms, smin, smax, qkv.shape[-1] - (hq + hk) * d)
        packed = out.view(batch, seq_len, -1)
        q = packed[..., : hq * d].unflatten(-1, (hq, d))
        k = packed[..., hq * d: (hq + hk) * d].unflatten(-1, (hk, d))
        v = packed[..., (hq + hk) * d:].unflatten(-1, (hk, d))
        res = c.attn_fwd(q, k, v, window, scale, softcap, doc_start, quant_out)
        o, lse = res[0], res[1]
        empty = qkv.new_empty(0)
        ctx.save_for_backward(x2, qkv, out, o, lse, cos if cos is not None else empty, sin if sin is not None else empty,
                              qs if qs is not None else empty, ks if ks is not None else empty, wqt, wsft)
        ctx.cfg, ctx.doc_start, ctx.weights = cfg, doc_start, weights
        ctx.flags = (cos is not None, q_scale is not None)
        ctx.meta = (x.shape, x.dtype, tuple(w.shape))
        ctx.scale_shapes = (None if q_scale is None else (q_scale.shape, q_scale.dtype),
                            None if k_scale is None else (k_scale.shape, k_scale.dtype))
        if quant_out:                             # MXFP8 copy of the attention output, written by the kernel's epilogue
            ctx.mark_non_differentiable(res[2], res[3])
            return o, res[2], res[3]
        return o, None, None

    @staticmethod
    def backward(ctx, d_out: Tensor, _dq=None, _dsf=None):
        c = co.ext()
        x2, qkv, out, o, lse, cos, sin, qs, ks, wqt, wsft = ctx.saved_tensors
        batch, seq_len, hq, hk, d, eps, rms, smin, smax, window, scale, softcap, _ = ctx.cfg
        has_rope, has_norm = ctx.flags
        x_shape, x_dtype, w_shape = ctx.meta
        packed = out.view(batch, seq_len, -1)
        q = packed[..., : hq * d].unflatten(-1, (hq, d))
        k = packed[..., hq * d: (hq + hk) * d].unflatten(-1, (hk, d))
        v = packed[..., (hq + hk) * d:].unflatten(-1, (hk, d))
        d_out = d_out if (d_out.dtype == BF16 and d_out.is_contiguous()) else d_out.to(BF16).contiguous()
        grad = torch.empty_like(packed)
        dk = grad[..., hq * d: (hq + hk) * d].unflatten(-1, (hk, d))
        dv = grad[..., (hq + hk) * d:].unflatten(-1, (hk, d))
        dq32 = c.attn_bwd(q, k, v, o, d_out, lse, dk, dv, window, scale, softcap, ctx.doc_start)
        g2 = grad.view(batch * seq_len, -1)
        need_dx = ctx.needs_input_grad[0]
        res = c.rope_qknorm_bwd(qkv, g2, g2, cos if has_rope else None, sin if has_rope else None, qs if has_norm else None,
                                ks if has_norm else None, seq_len, hq, hk, d, eps, rms, smin, smax, dq32.view(batch * seq_len, -1),
                                quantize=need_dx)
        dscale = res[0]
        dx = None
        if need_dx:
            gq, gsf = res[1], res[2]
            dx = torch.empty_like(x2)
            c.gemm_mxfp8(gq, gsf, wqt, wsft, dx)
            dx = dx.view(x_shape).to(x_dtype)
        grads = _weight_grads(c, g2, x2, ctx.weights, w_shape, ctx.needs_input_grad[9:])
        dqs = dks = None
        if has_norm:
            (qshape, qdt), (kshape, kdt) = ctx.scale_shapes
            dqs, dks = dscale[:hq].reshape(qshape).to(qdt), dscale[hq:].reshape(kshape).to(kdt)
        return (dx, None, None, None, None, dqs, dks, None, None) + tuple(grads)


def qkv_rope_attention(x: Tensor, weights: Sequence[Tensor], cos, sin, q_scale, k_scale, batch: int, seq_len: int, hq: int, hk: int,
                       d: int, eps: float, rms: bool, smin: float, smax: float, window: Optional[int], scale: Optional[float],
                       softcap: float = 0.0, doc_start: Optional[Tensor] = None, quantize_out: bool = False) -> Optional[Tensor]:
    """x [batch, seq_len, hidden] -> attention output [batch, seq_len, hq, 64]; None when the projection shape is not covered.
    `quantize_out`: an MXFP8 projection consumes the output; its quantised copy then comes attached as `.mxq`."""
    k_dim, n = weights[0].shape[1], sum(w.shape[0] for w in weights)
    if not supported(k_dim, n) or n % 32:
        return None
    smin, smax = max(smin, -3.0e38), min(smax, 3.0e38)
    w = seq_len if window is None else int(window)
    quant = bool(quantize_out and (hq * 64) % 128 == 0)
    cfg = (batch, seq_len, hq, hk, d, eps, rms, smin, smax, w, d ** -0.5 if scale is None else float(scale), float(softcap), quant)
    co.count_path("attention:tcgen05")
    xq, xsf = _attached_copy(x)
    o, oq, osf = _MXFP8QKVAttentionFn.apply(x, xq, xsf, cos, sin, q_scale, k_scale, cfg, doc_start, *weights)
    if quant:
        o.mxq = (oq, osf)
    return o


class _MXFP8MoEExpertsFn(torch.autograd.Function):
    """Same data flow as the bf16 expert function; the four grouped forward / input-gradient GEMMs read e4m3 operands that the
    gather, activation and combine-backward kernels emitted next to their bf16 outputs."""

    @staticmethod
    def forward(ctx, hidden: Tensor, gates: Tensor, top_idx: Tensor, activation: str, num_experts: int, *weights: Tensor):
        c = co.ext()
        up, down = weights[:num_experts], weights[num_experts:]
        top_k = top_idx.shape[1]
        h2 = co._as_bf16_2d(hidden)
        gates32 = gates.detach().float().contiguous()
        dest, src_of_row, seg_ends, counts, tile_expert, meta = c.route(top_idx.contiguous(), num_experts)
        packed, pq, psf = c.gather_rows(h2, src_of_row, meta, top_k, quantize=True)
        w_up, uq, usf, uqt, usft = _quantized_weight(up, stack=True)
        w_down, dq, dsf, dqt, dsft = _quantized_weight(down, stack=True)
        cap = packed.shape[0]
        pre = torch.empty((cap, w_up.shape[1]), dtype=BF16, device=hidden.device)
        c.gemm_mxfp8(pq, psf, uq, usf, pre, 1.0, tile_expert, meta)
        act, aq, asf = c.activation_fwd(pre, activation, meta, quantize=True)
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
        d2 = co._as_bf16_2d(dout)
        dy, dgates, gq, gsf = c.combine_bwd(d2, y, src_of_row, gates32, meta, quantize=True)
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
        need_dx = ctx.needs_input_grad[0]
        res = c.activation_bwd(dact, pre, ctx.activation, meta, quantize=need_dx)
        dpre = res[0]
        wgrad(dpre, packed, up, 0)
        dhidden = None
        if need_dx:
            dpacked = torch.empty_like(packed)
            c.gemm_mxfp8(res[1], res[2], uqt, usft, dpacked, 1.0, tile_expert, meta)
            dhidden = c.combine_fwd(dpacked, dest, None, gates32.shape[1]).view(shape).to(dtype)
        return (dhidden, dgates.to(gdtype), None, None, None) + tuple(grads)


def mxfp8_moe_experts(hidden, top_idx, gates, up_weights, down_weights, activation):
    d, h_up = up_weights[0].shape[1], up_weights[0].shape[0]
    h_down = down_weights[0].shape[1]
    if not (supported(d, h_up) and supported(h_down, down_weights[0].shape[0])):
        return co._MoEExpertsFn.apply(hidden, gates, top_idx, activation, len(up_weights), *up_weights, *down_weights)
    return _MXFP8MoEExpertsFn.apply(hidden, gates, top_idx, activation, len(up_weights), *up_weights, *down_weights)
