"""Op entry points used by the model.

One function per op.  CUDA tensors go to the sm_100a kernels in `cuda_ops` (and fail loudly if
the extension is not built); CPU tensors go to the plain-PyTorch definitions in `reference`,
which are also the oracle of the GPU tests.

Shapes the kernels do not cover stay correct through library or torch ops, and every such call is
counted in `cuda_ops.path_counts()` under a name that says which one ran, so a benchmark record can
show that none did:
  attention   head widths other than 64 / 128x64, padding masks, non-causal -> flash-attn or torch SDPA
              (`ops/attention_cuda.py`)
  linear      row pitch not a multiple of 16 bytes (k or n not a multiple of 8)  -> torch `F.linear`
  rms_norm    widths other than 128*{1,2,4,6,8,12,16}, other dtypes               -> torch ops
  cross_entropy on materialised logits (evaluation)                              -> torch ops
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor

from . import reference as ref


def _cuda():
    from . import cuda_ops
    return cuda_ops


def _pad_to(x: Tensor, dim: int, multiple: int) -> Tensor:
    size = x.shape[dim]
    pad = (-size) % multiple
    if pad == 0:
        return x
    shape = list(x.shape)
    shape[dim] = pad
    return torch.cat((x, x.new_zeros(shape)), dim=dim)


class _MXFP8LinearEmulated(torch.autograd.Function):
    """CPU emulation of the MXFP8 linear: forward blocks along K; dgrad blocks dY and W along N;
    wgrad blocks dY and X along the token dimension.  Zero padding to multiples of 32 does not
    change any block's amax, so padded and unpadded results agree."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor) -> Tensor:
        ctx.save_for_backward(x, weight)
        x2 = x.reshape(-1, x.shape[-1])
        y = ref.mxfp8_linear(_pad_to(x2, 1, 32), _pad_to(weight, 1, 32))
        return y.to(x.dtype).reshape(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, grad: Tensor):
        x, weight = ctx.saved_tensors
        x2 = x.reshape(-1, x.shape[-1]).float()
        g2 = grad.reshape(-1, grad.shape[-1]).float()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gq = ref.mxfp8_roundtrip(_pad_to(g2, 1, 32), -1)
            wq = ref.mxfp8_roundtrip(_pad_to(weight.float(), 0, 32), 0)
            gx = (gq @ wq).to(x.dtype).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            gq = ref.mxfp8_roundtrip(_pad_to(g2, 0, 32), 0)
            xq = ref.mxfp8_roundtrip(_pad_to(x2, 0, 32), 0)
            gw = (gq.t() @ xq).to(weight.dtype)
        return gx, gw


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor], precision: str = "default") -> Tensor:
    if x.is_cuda:
        return _cuda().linear(x, weight, bias, precision)
    if precision in ("mxfp8", "fp8"):
        y = _MXFP8LinearEmulated.apply(x, weight)
        return y if bias is None else y + bias.to(y.dtype)
    return F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))


def activate(x: Tensor, name: str) -> Tensor:
    return ref.activate(x, name)


def rms_norm(x: Tensor, weight: Optional[Tensor], eps: float) -> Tensor:
    if x.is_cuda:
        return _cuda().rms_norm(x, weight, eps)
    return ref.rms_norm(x, weight, eps)


def residual_rms_norm(x: Tensor, branch: Tensor, alpha: Optional[Tensor], beta: Optional[Tensor], weight: Optional[Tensor],
                      eps: float, quantize_out: bool = False) -> Tuple[Tensor, Tensor]:
    """x_new = alpha*x + beta*branch (alpha/beta None = 1) and rmsnorm(x_new); returns (x_new, normed).  `quantize_out` tells
    the GPU kernel that an MXFP8 projection consumes `normed`, so it writes the quantised copy in the same pass."""
    if x.is_cuda:
        return _cuda().residual_rms_norm(x, branch, alpha, beta, weight, eps, quantize_out)
    x_new = (x if alpha is None else alpha * x) + (branch if beta is None else beta * branch).to(x.dtype)
    return x_new, ref.rms_norm(x_new, weight, eps)


def rope_qk_norm(q, k, cos, sin, q_scale, k_scale, eps, rms, scale_min, scale_max):
    if q.is_cuda:
        return _cuda().rope_qk_norm(q, k, cos, sin, q_scale, k_scale, eps, rms, scale_min, scale_max)
    return ref.rope_qk_norm(q, k, cos, sin, q_scale, k_scale, eps, rms, scale_min, scale_max)


def attention(q, k, v, *, causal=True, window=None, scale=None, softcap_value=0.0, tanh_backend="exact",
              attn_mask=None, document_ids=None):
    """q[B,T,H,Dk], k[B,T,Hkv,Dk], v[B,T,Hkv,Dv] -> [B,T,H,Dv].  `window` may be an int, a 0-dim
    int tensor (device-resident so the schedule can change it without a host sync) or None."""
    if q.is_cuda:
        return _cuda().attention(q, k, v, causal=causal, window=window, scale=scale,
                                 softcap_value=softcap_value, tanh_backend=tanh_backend,
                                 attn_mask=attn_mask, document_ids=document_ids)
    w = int(window) if window is not None else None
    return ref.attention(q, k, v, causal=causal, window=w, scale=scale, softcap_value=softcap_value,
                         tanh_backend=tanh_backend, attn_mask=attn_mask, document_ids=document_ids)


def router(logits: Tensor, top_k: int, full_softmax: bool, want_balance: bool, num_experts: int):
    """Router decisions from logits [tokens, experts]: (top_idx [T, k], gates fp32 [T, k], balance loss or None).
    fp32 softmax; top-1 / full-softmax gates are the chosen experts' probabilities, otherwise the softmax renormalised over the
    selection; balance = E * sum_e f_e * mean_prob_e (reference `model/feedforward/moe.py:55-88`)."""
    if logits.is_cuda:
        return _cuda().router(logits, top_k, full_softmax, want_balance, num_experts)
    top_idx, gates, probs = ref.router_gates(logits, top_k, full_softmax)
    return top_idx, gates, (ref.load_balance_loss(probs, top_idx, num_experts) if want_balance else None)


def moe_experts(hidden: Tensor, top_idx: Tensor, gates: Tensor, up_weights: Sequence[Tensor],
                down_weights: Sequence[Tensor], up_biases, down_biases, activation: str,
                up_precision: str, down_precision: str) -> Tensor:
    """Dropless expert computation for tokens hidden[M,d] with choices top_idx[M,k], gates[M,k].

    sort by expert -> grouped up GEMM -> activation -> grouped down GEMM -> inverse gather ->
    gate-weighted sum over k (reference `model/feedforward/moe.py:94-134`).
    """
    if hidden.is_cuda:
        return _cuda().moe_experts(hidden, top_idx, gates, up_weights, down_weights, up_biases, down_biases,
                                   activation, up_precision, down_precision)
    num_experts, top_k = len(up_weights), top_idx.shape[1]
    expert_ids, order, inverse, offsets = ref.counted_expert_routing(top_idx, num_experts)
    packed = hidden[order // top_k]
    ends = offsets.tolist()

    def grouped(x, weights, biases, precision):
        pieces, start = [], 0
        for e, end in enumerate(ends):
            pieces.append(linear(x[start:end], weights[e], None if biases is None else biases[e], precision))
            start = end
        return torch.cat(pieces, dim=0)

    packed = grouped(packed, up_weights, up_biases, up_precision)
    packed = ref.activate(packed, activation)
    packed = grouped(packed, down_weights, down_biases, down_precision)
    return ref.combine_expert_outputs(packed, inverse, gates).to(hidden.dtype)


def cross_entropy(logits: Tensor, targets: Tensor, ignore_index: int = -100) -> Tensor:
    if logits.is_cuda:
        return _cuda().cross_entropy(logits, targets, ignore_index)
    return ref.cross_entropy(logits, targets, ignore_index)


def linear_cross_entropy(x: Tensor, weight: Tensor, targets: Tensor, ignore_index: int = -100) -> Tensor:
    if x.is_cuda:
        return _cuda().linear_cross_entropy(x, weight, targets, ignore_index)
    return ref.linear_cross_entropy(x, weight, targets, ignore_index)
