"""Front end of the tcgen05 attention kernels (`csrc/attention`): causal, optionally sliding-window; value heads 64 wide,
query / key heads 64 wide or 128 wide (multi-head latent attention: content + rotary parts)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor


def supported(q: Tensor, k: Tensor, v: Tensor, softcap_value: float) -> bool:
    b, t, h, d = q.shape
    return (q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 and d in (64, 128) and k.shape[-1] == d
            and v.shape[-1] == 64 and t % 128 == 0 and softcap_value >= 0.0 and h % k.shape[2] == 0
            and all(x.stride(3) == 1 and x.stride(2) == x.shape[3] and x.stride(0) == t * x.stride(1) and x.stride(1) % 8 == 0 for x in (q, k, v)))


def document_starts(document_ids: Tensor) -> Tensor:
    """[B, T] document ids that are constant on contiguous runs of tokens (the loader's cumulative end-of-sequence count)
    -> int32 [B, T]: position of the first token of each token's document.  With it, "same document" is the per-row
    look-back bound `key >= start[query]`, which the kernels fold into the sliding-window test."""
    b, t = document_ids.shape
    idx = torch.arange(t, device=document_ids.device).expand(b, t)
    new = torch.ones_like(document_ids, dtype=torch.bool)
    new[:, 1:] = document_ids[:, 1:] != document_ids[:, :-1]
    return torch.where(new, idx, torch.zeros_like(idx)).cummax(dim=1).values.to(torch.int32).contiguous()


class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, v: Tensor, window: int, scale: float, softcap: float, doc_start: Optional[Tensor]) -> Tensor:
        from .cuda_ops import ext
        out, lse = ext().attn_fwd(q, k, v, window, scale, softcap, doc_start)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (window, scale, softcap)
        ctx.doc_start = doc_start
        return out

    @staticmethod
    def backward(ctx, d_out: Tensor):
        from .cuda_ops import ext
        q, k, v, out, lse = ctx.saved_tensors
        window, scale, softcap = ctx.cfg
        b, t, h, d = q.shape
        hk = k.shape[2]
        d_out = d_out if (d_out.stride(3) == 1 and d_out.stride(2) == 64 and d_out.stride(0) == t * d_out.stride(1)) else d_out.contiguous()
        if d != 64:                   # wide query / key heads: separate gradient tensors
            dk = torch.empty((b, t, hk, d), dtype=q.dtype, device=q.device)
            dv = torch.empty((b, t, hk, 64), dtype=q.dtype, device=q.device)
            dq32 = ext().attn_bwd(q, k, v, out, d_out, lse, dk, dv, window, scale, softcap, ctx.doc_start)
            return dq32.to(q.dtype), dk, dv, None, None, None, None
        # one packed gradient buffer [B, T, (H + 2 Hkv) * 64]: dk and dv are written in place by the kernel, dq is converted into it
        packed = torch.empty((b, t, (h + 2 * hk) * d), dtype=q.dtype, device=q.device)
        dk = packed[..., h * d: (h + hk) * d].unflatten(-1, (hk, d))
        dv = packed[..., (h + hk) * d:].unflatten(-1, (hk, d))
        dq32 = ext().attn_bwd(q, k, v, out, d_out, lse, dk, dv, window, scale, softcap, ctx.doc_start)
        dq = packed[..., : h * d].unflatten(-1, (h, d))
        dq.copy_(dq32)
        return dq, dk, dv, None, None, None, None


def attention(q: Tensor, k: Tensor, v: Tensor, *, window: Optional[int], scale: Optional[float], softcap: float = 0.0,
              document_ids: Optional[Tensor] = None) -> Tensor:
    """`softcap` > 0 caps the scaled logits with softcap * tanh(logit / softcap) (hardware `tanh.approx`) before the softmax;
    `document_ids` [B, T] (constant on contiguous runs) restricts every query to keys of its own document."""
    t, d = q.shape[1], q.shape[3]
    doc_start = None if document_ids is None else document_starts(document_ids)
    return _AttentionFn.apply(q, k, v, t if window is None else int(window), d ** -0.5 if scale is None else float(scale), float(softcap),
                              doc_start)
