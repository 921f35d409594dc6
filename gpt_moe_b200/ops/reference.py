"""Plain-PyTorch definitions of every op in the framework.

These functions are (a) the execution path on CPU, where they run in fp32 under autograd, and
(b) the oracle every CUDA kernel in `csrc/` is tested against.  They are written for clarity,
not speed, and use only differentiable torch operations so their gradients come from autograd.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor

# --------------------------------------------------------------------------------------------
# normalisation
# --------------------------------------------------------------------------------------------

def rms_norm(x: Tensor, weight: Optional[Tensor], eps: float) -> Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * weight, statistics in fp32."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


def residual_rms_norm(x: Tensor, branch: Tensor, beta: Tensor, alpha: Optional[Tensor],
                      weight: Tensor, eps: float) -> Tuple[Tensor, Tensor]:
    """x_new = alpha*x + beta*branch ; y = rms_norm(x_new).  Returns (x_new, y).

    Reference counterpart: `experiments/057-fused-attention-residual-rmsnorm.patch`.
    """
    x_new = (x if alpha is None else alpha * x) + beta * branch.to(x.dtype)
    return x_new, rms_norm(x_new, weight, eps)


# --------------------------------------------------------------------------------------------
# rotary embedding and QK-norm.  Layout here is [B, T, H, D] (token-major, head-minor).
# --------------------------------------------------------------------------------------------

def rope_tables(head_size: int, base_theta: float, max_seq_len: int, device=None) -> Tuple[Tensor, Tensor]:
    """fp32 cos/sin tables of shape [max_seq_len, head_size/2] (reference `model/position/rotary.py:10-29`)."""
    inv_freq = 1.0 / (base_theta ** (torch.arange(0, head_size, 2, dtype=torch.float32, device=device) / head_size))
    freqs = torch.outer(torch.arange(max_seq_len, dtype=torch.float32, device=device), inv_freq)
    return freqs.cos(), freqs.sin()


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Interleaved-pair rotation: (x0,x1),(x2,x3),... of x[B,T,H,D]; cos/sin [T, D/2]."""
    b, t, h, d = x.shape
    pairs = x.reshape(b, t, h, d // 2, 2)
    x1, x2 = pairs[..., 0], pairs[..., 1]
    c = cos[:t].to(x.dtype)[None, :, None, :]
    s = sin[:t].to(x.dtype)[None, :, None, :]
    return torch.stack((x1 * c - x2 * s, x1 * s + x2 * c), dim=-1).reshape(b, t, h, d)


def qk_norm(x: Tensor, scale: Tensor, eps: float, rms: bool, scale_min: float, scale_max: float) -> Tensor:
    """Per-head normalisation of x[B,T,H,D] with a learned, clamped per-head scale[H].

    gain = rsqrt(mean|sum(x^2) + eps) computed from x in its own dtype then cast back
    (reference `model/attention/self_attention.py:212-247`).
    """
    sq = x.pow(2)
    stat = sq.mean(dim=-1, keepdim=True) if rms else sq.sum(dim=-1, keepdim=True)
    gain = torch.rsqrt(stat + eps).to(x.dtype)
    s = torch.clamp(scale.reshape(1, 1, -1, 1), min=scale_min, max=scale_max).to(x.dtype)
    return x * gain * s


def rope_qk_norm(q: Tensor, k: Tensor, cos: Optional[Tensor], sin: Optional[Tensor],
                 q_scale: Optional[Tensor], k_scale: Optional[Tensor], eps: float, rms: bool,
                 scale_min: float, scale_max: float) -> Tuple[Tensor, Tensor]:
    """RoPE first, then QK-norm over the rotated values (order as in the reference's fused kernels,
    `model/attention/qk_norm_rope.py:59-66`)."""
    if cos is not None:
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    if q_scale is not None:
        q = qk_norm(q, q_scale, eps, rms, scale_min, scale_max)
        k = qk_norm(k, k_scale, eps, rms, scale_min, scale_max)
    return q, k


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------

def softcap(scores: Tensor, cap: float, backend: str = "exact") -> Tensor:
    """cap * tanh(scores / cap) with the four tanh variants of the reference
    (`model/attention/logit_softcapping.py`): "exact"/"ptx" use tanh ("ptx" is `tanh.approx.f32`
    on the GPU, exact here), "clamp" is a hard clip, "rational" is z(27+z^2)/(27+9z^2)
    with z clipped to [-3, 3], where the expression reaches exactly +-1."""
    if cap <= 0:
        return scores
    z = scores / cap
    if backend == "clamp":
        t = z.clamp(-1.0, 1.0)
    elif backend == "rational":
        z = z.clamp(-3.0, 3.0)
        z2 = z * z
        t = z * (27.0 + z2) / (27.0 + 9.0 * z2)
    else:
        t = torch.tanh(z)
    return cap * t


def attention_mask(seq_len: int, device, causal: bool, window: Optional[int],
                   attn_mask: Optional[Tensor] = None, document_ids: Optional[Tensor] = None) -> Optional[Tensor]:
    """Boolean keep-mask [B or 1, 1, T, T].

    causal: q >= k.  window (inclusive, W+1 keys): q - k <= W, or |q - k| <= W for encoders
    (reference `model/gpt.py:360-372`).  attn_mask [B,T] marks valid (non-padding) tokens; both
    ends must be valid.  document_ids [B,T]: both ends in the same document.
    """
    need = causal or window is not None or attn_mask is not None or document_ids is not None
    if not need:
        return None
    q = torch.arange(seq_len, device=device)[:, None]
    k = torch.arange(seq_len, device=device)[None, :]
    keep = torch.ones(seq_len, seq_len, dtype=torch.bool, device=device)
    if causal:
        keep &= q >= k
    if window is not None:
        keep &= ((q - k) <= window) if causal else ((q - k).abs() <= window)
    keep = keep[None, None]
    if attn_mask is not None:
        am = attn_mask.bool()
        keep = keep & (am[:, None, :, None] & am[:, None, None, :])
    if document_ids is not None:
        keep = keep & (document_ids[:, None, :, None] == document_ids[:, None, None, :])
    return keep


def attention(q: Tensor, k: Tensor, v: Tensor, *, causal: bool = True, window: Optional[int] = None,
              scale: Optional[float] = None, softcap_value: float = 0.0, tanh_backend: str = "exact",
              attn_mask: Optional[Tensor] = None, document_ids: Optional[Tensor] = None) -> Tensor:
    """Scaled dot-product attention on q[B,T,H,Dk], k[B,T,Hkv,Dk], v[B,T,Hkv,Dv] -> [B,T,H,Dv].

    Rows whose mask is empty (padding queries) produce zeros.  Softmax in fp32.
    """
    b, t, h, dk = q.shape
    hkv = k.shape[2]
    if hkv != h:
        rep = h // hkv
        k = k.repeat_interleave(rep, dim=2)
        v = v.repeat_interleave(rep, dim=2)
    scale = dk ** -0.5 if scale is None else scale
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    s = softcap(s, softcap_value, tanh_backend)
    keep = attention_mask(t, q.device, causal, window, attn_mask, document_ids)
    if keep is not None:
        s = s.masked_fill(~keep, float("-inf"))
        empty = ~keep.any(dim=-1, keepdim=True)
        s = s.masked_fill(empty, 0.0)
    p = torch.softmax(s, dim=-1)
    if keep is not None:
        p = p.masked_fill(empty, 0.0)
    return torch.einsum("bhqk,bkhd->bqhd", p, v.float()).to(q.dtype)


# --------------------------------------------------------------------------------------------
# mixture of experts
# --------------------------------------------------------------------------------------------

def counted_expert_routing(indices: Tensor, num_experts: int) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    """Stable bucket sort of the flattened top-k expert choices.

    Returns (expert_indices sorted, order, inverse_order, offsets) where `order[j]` is the flat
    (token*k + slot) index that lands in packed row j, `inverse_order` its inverse, and
    `offsets[e]` (int32) the cumulative END of expert e's segment.  Within a segment the original
    order is preserved (reference `model/feedforward/routing.py:62-96`).
    """
    flat = indices.reshape(-1)
    order = torch.sort(flat, stable=True).indices
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(order.numel(), device=order.device, dtype=order.dtype)
    counts = torch.bincount(flat, minlength=num_experts)[:num_experts]
    offsets = counts.cumsum(0).to(torch.int32)
    return flat[order], order, inverse, offsets


def grouped_linear(x: Tensor, weight: Tensor, offsets: Tensor) -> Tensor:
    """Ragged grouped GEMM: rows offsets[e-1]:offsets[e] of x[Mk,K] times weight[e] ([E,N,K]) transposed."""
    out = x.new_zeros(x.shape[0], weight.shape[1])
    ends = offsets.tolist()
    start = 0
    pieces = []
    for e, end in enumerate(ends):
        pieces.append(x[start:end] @ weight[e].to(x.dtype).t())
        start = end
    return torch.cat(pieces, dim=0) if pieces else out


def activate(x: Tensor, name: str) -> Tensor:
    """gelu | relu | relu2 | silu | swiglu (gate = first half; reference `model/feedforward/mlp.py:55-75`)."""
    if name == "gelu":
        return F.gelu(x)
    if name == "relu":
        return F.relu(x)
    if name == "relu2":
        return F.relu(x) ** 2
    if name == "silu":
        return F.silu(x)
    if name == "swiglu":
        g, u = x.chunk(2, dim=-1)
        return F.silu(g) * u
    raise ValueError(f"unsupported activation function: {name}")


def combine_expert_outputs(packed: Tensor, inverse_order: Tensor, gates: Tensor) -> Tensor:
    """out[t] = sum_k gates[t,k] * packed[inverse_order[t*k_+k]] (reference `model/feedforward/moe.py:133-134`)."""
    m, k = gates.shape
    y = packed[inverse_order].view(m, k, -1)
    return (y * gates[:, :, None].to(y.dtype)).sum(dim=1)


def router_gates(logits: Tensor, top_k: int, full_softmax: bool) -> Tuple[Tensor, Tensor, Tensor]:
    """fp32 router: top-k indices, gate weights, and full-softmax probabilities.

    top-1 (or `full_softmax`): gate = full-softmax probability of the chosen expert (not 1.0);
    otherwise softmax renormalised over the selected logits (reference `model/feedforward/moe.py:59-76`).
    """
    logits = logits.float()
    if top_k == 1:
        top_logits, top_idx = logits.max(dim=-1, keepdim=True)          # same choice as topk, one small reduction instead of a sort
    else:
        top_logits, top_idx = torch.topk(logits, top_k, dim=-1)
    probs = F.softmax(logits, dim=-1)
    if top_k == 1 or full_softmax:
        gates = probs.gather(-1, top_idx)
    else:
        gates = F.softmax(top_logits, dim=-1)
    return top_idx, gates, probs


def load_balance_loss(probs: Tensor, top_idx: Tensor, num_experts: int) -> Tensor:
    """Switch-style E * sum_e f_e * mean_prob_e with f_e = routed fraction (reference `model/feedforward/moe.py:78-88`)."""
    mean_probs = probs.mean(dim=0)
    counts = torch.zeros_like(mean_probs).scatter_add_(
        0, top_idx.reshape(-1), torch.ones(top_idx.numel(), dtype=mean_probs.dtype, device=probs.device))
    return num_experts * ((counts / top_idx.numel()) * mean_probs).sum()


# --------------------------------------------------------------------------------------------
# loss
# --------------------------------------------------------------------------------------------

def cross_entropy(logits: Tensor, targets: Tensor, ignore_index: int = -100) -> Tensor:
    """Mean fp32 cross-entropy over rows whose target != ignore_index."""
    return F.cross_entropy(logits.float(), targets, ignore_index=ignore_index, reduction="mean")


def linear_cross_entropy(x: Tensor, weight: Tensor, targets: Tensor, ignore_index: int = -100) -> Tensor:
    """LM head + cross-entropy as one op (the CUDA version never materialises the logits)."""
    return cross_entropy(F.linear(x, weight.to(x.dtype)), targets, ignore_index)


# --------------------------------------------------------------------------------------------
# MXFP8 emulation: e4m3 payload, one E8M0 (power-of-two) scale per 32 consecutive elements.
# --------------------------------------------------------------------------------------------

E4M3_MAX = 448.0
MX_BLOCK = 32


def e8m0_scale_from_amax(amax: Tensor) -> Tensor:
    """Power-of-two scale 2^ceil(log2(amax/448)) by integer arithmetic on the fp32 bits.

    Same rule as the reference `model/linear/fp8/custom/quantization.py:5-13`: round the mantissa
    up into the exponent, floor at 2^-126, amax == 0 -> 1, NaN/inf -> 0.
    """
    s = (amax.float() / E4M3_MAX).contiguous()
    bits = s.view(torch.int32)
    bits = (bits + 0x007FFFFF) & 0x7F800000
    bits = torch.clamp(bits, min=0x00800000)
    out = bits.view(torch.float32)
    out = torch.where(amax == 0, torch.ones_like(out), out)
    return torch.where(torch.isfinite(amax.float()), out, torch.zeros_like(out))


def mxfp8_quantize(x: Tensor, dim: int = -1) -> Tuple[Tensor, Tensor]:
    """Quantise along `dim` in blocks of 32.  Returns (payload float8_e4m3fn with x's shape,
    scales fp32 with the blocked dimension divided by 32).  `dim` must be a multiple of 32."""
    xm = x.float().movedim(dim, -1)
    shape = xm.shape
    blocks = xm.reshape(*shape[:-1], shape[-1] // MX_BLOCK, MX_BLOCK)
    scale = e8m0_scale_from_amax(blocks.abs().amax(dim=-1))
    q = (blocks / scale[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(shape).movedim(-1, dim), scale.movedim(-1, dim)


def mxfp8_dequantize(q: Tensor, scale: Tensor, dim: int = -1) -> Tensor:
    qm = q.float().movedim(dim, -1)
    sm = scale.movedim(dim, -1)
    shape = qm.shape
    out = qm.reshape(*shape[:-1], shape[-1] // MX_BLOCK, MX_BLOCK) * sm[..., None]
    return out.reshape(shape).movedim(-1, dim)


def mxfp8_roundtrip(x: Tensor, dim: int = -1) -> Tensor:
    """x quantised to MXFP8 along `dim` and expanded back to fp32 (what a block-scaled MMA multiplies)."""
    q, s = mxfp8_quantize(x, dim)
    return mxfp8_dequantize(q, s, dim)


def mxfp8_linear(x: Tensor, weight: Tensor) -> Tensor:
    """Emulated MXFP8 GEMM y = Q(x) Q(w)^T with both operands blocked along K, fp32 accumulate."""
    return (mxfp8_roundtrip(x, -1) @ mxfp8_roundtrip(weight, -1).t())


# --------------------------------------------------------------------------------------------
# Polar Express (Muon orthogonalisation)
# --------------------------------------------------------------------------------------------

# five coefficient triples for num_iters=5, safety_factor=2e-2, cushion=2 (arXiv:2505.16932;
# reference `optimizers/polar_express.py:380-387`)
POLAR_EXPRESS_COEFFS = (
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
)


def polar_express(g: Tensor, dtype: torch.dtype = torch.bfloat16) -> Tensor:
    """Approximate U V^T of g[..., m, n] by the five-step Polar Express iteration
    X <- a X + (b A + c A^2) X with A = X X^T, on the wide orientation, in `dtype`."""
    x = g.to(dtype)
    tall = g.size(-2) > g.size(-1)
    if tall:
        x = x.mT
    x = x / (x.norm(dim=(-2, -1), keepdim=True) * (1 + 2e-2) + 1e-6)
    for a, b, c in POLAR_EXPRESS_COEFFS:
        A = x @ x.mT
        B = b * A + c * (A @ A)
        x = a * x + B @ x
    return x.mT if tall else x


def newton_schulz5(g: Tensor, steps: int = 5, eps: float = 1e-7, dtype: torch.dtype = torch.bfloat16) -> Tensor:
    """Quintic Newton-Schulz with (3.4445, -4.7750, 2.0315) (reference `optimizers/muon.py:65-100`)."""
    a, b, c = 3.4445, -4.7750, 2.0315
    tall = g.size(0) > g.size(1)
    x = g.T if tall else g
    x = (x / (x.norm() + eps)).to(dtype)
    for _ in range(steps):
        A = x @ x.T
        B = A @ x
        x = a * x + b * B + c * (A @ B)
    x = x.T if tall else x
    return x.to(g.dtype)


def svd_orthogonalize(g: Tensor) -> Tensor:
    u, _, vh = torch.linalg.svd(g.float(), full_matrices=False)
    return (u @ vh).to(g.dtype)
