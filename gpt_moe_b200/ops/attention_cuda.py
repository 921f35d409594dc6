"""Attention on the GPU.

`attention()` takes token-major tensors q[B,T,H,Dk], k[B,T,Hkv,Dk], v[B,T,Hkv,Dv] (views into the
packed projection output are fine: only the last dimension must be contiguous).

Causal / sliding-window attention without a padding mask (with or without logit soft-capping and
document masking) goes to the tcgen05 kernel in `csrc/attention` when it is built for the head size;
everything else — and any shape the kernel does not cover — runs through the flash-attn library
kernel or torch's fused SDPA with an explicit boolean mask, which is the slow but general path.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F
from torch import Tensor

from . import reference as ref

_flash = None


def _flash_attn():
    """flash-attn (library) if it imports and runs on this GPU; probed once."""
    global _flash
    if _flash is None:
        try:
            from flash_attn import flash_attn_func
            q = torch.zeros(1, 128, 1, 64, device="cuda", dtype=torch.bfloat16)
            flash_attn_func(q, q, q, causal=True, window_size=(16, 0))
            torch.cuda.synchronize()
            _flash = flash_attn_func
        except Exception:
            _flash = False
    return _flash


def _window_int(window) -> Optional[int]:
    if window is None:
        return None
    host = getattr(window, "host_value", None)
    return int(host) if host is not None else int(window)


def attention(q: Tensor, k: Tensor, v: Tensor, *, causal: bool = True, window=None, scale: Optional[float] = None,
              softcap_value: float = 0.0, tanh_backend: str = "exact", attn_mask: Optional[Tensor] = None,
              document_ids: Optional[Tensor] = None) -> Tensor:
    b, t, h, dk = q.shape
    w = _window_int(window)
    if w is not None and w >= t - 1 and causal:
        w = None
    if attn_mask is None and causal:
        from . import attention_tc
        from .cuda_ops import count_path
        if attention_tc.supported(q, k, v, softcap_value):
            count_path("attention:tcgen05")
            return attention_tc.attention(q, k, v, window=w, scale=scale, softcap=softcap_value, document_ids=document_ids)
        flash = _flash_attn()
        dv = v.shape[-1]
        if document_ids is None and flash and q.dtype == torch.bfloat16 and dv <= dk and dk <= 256 and softcap_value == 0.0:
            # head sizes the tcgen05 kernel is not built for (e.g. MLA: 128-wide keys, 64-wide values) go to the library kernel;
            # it wants equal widths, so narrower values are zero-padded and the padding columns of the result dropped
            count_path("attention:flash_attn")
            vp = v if dv == dk else F.pad(v, (0, dk - dv))
            out = flash(q, k, vp, softmax_scale=scale if scale is not None else dk ** -0.5, causal=True,
                        window_size=(w, 0) if w is not None else (-1, -1))
            return out if dv == dk else out[..., :dv]
    from .cuda_ops import count_path
    count_path("attention:torch")
    if softcap_value > 0.0:
        return ref.attention(q, k, v, causal=causal, window=w, scale=scale, softcap_value=softcap_value,
                             tanh_backend=tanh_backend, attn_mask=attn_mask, document_ids=document_ids)
    keep = ref.attention_mask(t, q.device, causal, w, attn_mask, document_ids)
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    out = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=keep, is_causal=keep is None and causal, scale=scale,
                                         enable_gqa=k.shape[2] != h)
    return out.transpose(1, 2)
