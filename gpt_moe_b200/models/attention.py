"""Self-attention: MHA / GQA / MQA with RoPE, QK-norm, sliding window, document masking, softcap.

Parameter names (`q_proj, k_proj, v_proj, out_proj, q_scale, k_scale`) and shapes follow the
reference module (`model/attention/self_attention.py:57-116`) so checkpoints interchange.
Internally activations stay token-major `[B, T, H, D]` end to end: the projections write it, the
RoPE+QK-norm op updates it in place and the attention kernel reads it through strided tiles, so
the reference's `[B,H,T,D]` transposes (`self_attention.py:185-187, 265`) never happen.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
from torch import Tensor

from ..ops import api
from .linear import Linear
from .rotary import Rotary


@torch.no_grad()
def qk_scale_debug_string(model) -> str:
    """Largest raw and clamped Q/K scales over all blocks (reference `self_attention.py:25-54`)."""
    stats = [0.0, 0.0, 0.0, 0.0]
    for blk in model.transformer.h:
        attn = blk.attn
        if not hasattr(attn, "q_scale"):
            continue
        vals = (attn.q_scale.max(), attn.k_scale.max(),
                attn.q_scale.clamp(attn.qk_scale_min, attn.qk_scale_max).max(),
                attn.k_scale.clamp(attn.qk_scale_min, attn.qk_scale_max).max())
        stats = [max(s, float(v)) for s, v in zip(stats, vals)]
    return (f"max q_scale raw/eff: {stats[0]:.4f}/{stats[2]:.4f} | "
            f"max k_scale raw/eff: {stats[1]:.4f}/{stats[3]:.4f} | ")


class AttentionContext:
    """Per-forward attention inputs shared by all layers.

    window: 0-dim int32 tensor (device resident, so a window-schedule change is a `fill_`, not a
    new launch configuration) or None for full attention.
    """
    __slots__ = ("window", "attn_mask", "document_ids", "doc_start")

    def __init__(self, window: Optional[Tensor], attn_mask: Optional[Tensor], document_ids: Optional[Tensor]):
        self.window, self.attn_mask, self.document_ids = window, attn_mask, document_ids
        self.doc_start = None           # per-token start of its document, derived from document_ids on first use


class SelfAttention(nn.Module):
    def __init__(self, gpt_config, training_config, layer_idx: int = 0) -> None:
        super().__init__()
        self.hidden_size = gpt_config.hidden_size
        self.n_heads = gpt_config.n_heads
        self.is_full_attention = layer_idx in gpt_config.full_attention_layers
        if self.is_full_attention:
            self.attn_dim, self.n_kv_heads = gpt_config.global_attn_dim, gpt_config.global_n_kv_heads
        else:
            self.attn_dim, self.n_kv_heads = gpt_config.attn_dim, gpt_config.n_kv_heads
        assert 1 <= self.n_kv_heads <= self.n_heads and self.n_heads % self.n_kv_heads == 0, \
            "n_kv_heads must divide n_heads"
        assert self.attn_dim % self.n_heads == 0, "attn_dim must be divisible by n_heads"
        self.head_size = self.attn_dim // self.n_heads
        kv_dim = self.n_kv_heads * self.head_size
        self.q_proj = Linear(self.hidden_size, self.attn_dim, role="q_proj", bias=gpt_config.use_bias)
        self.k_proj = Linear(self.hidden_size, kv_dim, role="k_proj", bias=gpt_config.use_bias)
        self.v_proj = Linear(self.hidden_size, kv_dim, role="v_proj", bias=gpt_config.use_bias)
        self.out_proj = Linear(self.attn_dim, self.hidden_size, role="out_proj", bias=gpt_config.use_bias)

        theta = gpt_config.global_rope_theta if self.is_full_attention else gpt_config.rope_base_theta
        self.rotary = (Rotary(self.head_size, theta, training_config.max_seq_len)
                       if gpt_config.pos_encoding_type.lower() == "rope" else None)
        self.use_qk_norm = gpt_config.use_qk_norm
        self.qk_norm_type = gpt_config.qk_norm_type
        self.qk_scale_min, self.qk_scale_max = gpt_config.qk_scale_min, gpt_config.qk_scale_max
        self.qk_eps = gpt_config.qk_eps
        if self.use_qk_norm:
            self.q_scale = nn.Parameter(torch.full((1, self.n_heads, 1, 1), gpt_config.qk_scale_init))
            self.k_scale = nn.Parameter(torch.full((1, self.n_kv_heads, 1, 1), gpt_config.qk_scale_init))
        self.is_causal = gpt_config.is_causal
        self.use_flex_attention = gpt_config.use_flex_attention
        self.softcap = gpt_config.attn_logit_softcap if gpt_config.use_attn_logit_softcapping else 0.0
        self.tanh_backend = gpt_config.tanh_backend

    def project_qkv(self, x: Tensor):
        b, t, _ = x.shape
        d, hq, hk = self.head_size, self.n_heads, self.n_kv_heads
        if x.is_cuda and self.q_proj.bias is None and d in (32, 64, 128) and hq + hk <= 64:
            # one GEMM over the concatenated q/k/v weights, then RoPE + QK-norm in place on the packed rows
            from ..ops import cuda_ops
            qkv = cuda_ops.linear_multi(x, (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight), self.q_proj.precision)
            cos = sin = None
            if self.rotary is not None:
                cos, sin = self.rotary.cos_cached[:t], self.rotary.sin_cached[:t]
            qkv = cuda_ops.rope_qk_norm_packed(
                qkv.view(b * t, -1), cos, sin, self.q_scale if self.use_qk_norm else None,
                self.k_scale if self.use_qk_norm else None, t, hq, hk, d, self.qk_eps, self.qk_norm_type == "rms",
                self.qk_scale_min, self.qk_scale_max).view(b, t, -1)
            return cuda_ops.split_qkv(qkv, hq, hk, d)
        q = self.q_proj(x).view(b, t, self.n_heads, self.head_size)
        k = self.k_proj(x).view(b, t, self.n_kv_heads, self.head_size)
        v = self.v_proj(x).view(b, t, self.n_kv_heads, self.head_size)
        cos = sin = None
        if self.rotary is not None:
            cos, sin = self.rotary.cos_cached[:t], self.rotary.sin_cached[:t]
        q, k = api.rope_qk_norm(
            q, k, cos, sin,
            self.q_scale if self.use_qk_norm else None, self.k_scale if self.use_qk_norm else None,
            self.qk_eps, self.qk_norm_type == "rms", self.qk_scale_min, self.qk_scale_max)
        return q, k, v

    def _fused_rope_attention(self, x: Tensor, ctx: AttentionContext) -> Optional[Tensor]:
        """One QKV GEMM, then RoPE + QK-norm + causal / sliding-window attention as a single autograd node (CUDA, 64-wide heads,
        optional logit soft-capping and document masking, no padding mask).  Returns None when the shapes or options call for the general path."""
        b, t, _ = x.shape
        d, hq, hk = self.head_size, self.n_heads, self.n_kv_heads
        if not (x.is_cuda and self.q_proj.bias is None and d == 64 and hq + hk <= 64 and hq % hk == 0 and t % 128 == 0
                and self.is_causal and ctx.attn_mask is None):
            return None
        from ..ops import cuda_ops
        from ..ops.attention_cuda import _window_int
        cos = sin = None
        if self.rotary is not None:
            cos, sin = self.rotary.cos_cached[:t], self.rotary.sin_cached[:t]
        window = None if (self.is_full_attention or not self.use_flex_attention) else _window_int(ctx.window)
        doc_start = None
        if ctx.document_ids is not None:
            if getattr(ctx, "doc_start", None) is None:          # computed once per forward pass, shared by all layers
                from ..ops.attention_tc import document_starts
                ctx.doc_start = document_starts(ctx.document_ids)
            doc_start = ctx.doc_start
        weights = (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight)
        if self.q_proj.precision in ("mxfp8", "fp8"):
            # MXFP8 projection: one autograd node from the projection to the attention output, so the backward's RoPE kernel
            # hands the quantised dQKV rows straight to the input-gradient GEMM
            from ..ops import mxfp8
            y = mxfp8.qkv_rope_attention(
                x, weights, cos, sin, self.q_scale if self.use_qk_norm else None, self.k_scale if self.use_qk_norm else None,
                b, t, hq, hk, d, self.qk_eps, self.qk_norm_type == "rms", self.qk_scale_min, self.qk_scale_max, window, None,
                self.softcap, doc_start, quantize_out=self.out_proj.precision in ("mxfp8", "fp8"))
            if y is not None:
                return y
        qkv = cuda_ops.linear_multi(x, weights, self.q_proj.precision)
        return cuda_ops.rope_attention_packed(
            qkv.view(b * t, -1), cos, sin, self.q_scale if self.use_qk_norm else None, self.k_scale if self.use_qk_norm else None,
            b, t, hq, hk, d, self.qk_eps, self.qk_norm_type == "rms", self.qk_scale_min, self.qk_scale_max, window, None, self.softcap, doc_start)

    def forward(self, x: Tensor, ctx: AttentionContext) -> Tensor:
        b, t, _ = x.shape
        y = self._fused_rope_attention(x, ctx)
        if y is not None:
            merged = y.reshape(b, t, self.attn_dim)
            if getattr(y, "mxq", None) is not None:           # MXFP8 copy written by the attention kernel's epilogue
                merged.mxq = y.mxq
            return self.out_proj(merged)
        q, k, v = self.project_qkv(x)
        y = api.attention(
            q, k, v, causal=self.is_causal,
            window=None if (self.is_full_attention or not self.use_flex_attention) else ctx.window,
            softcap_value=self.softcap, tanh_backend=self.tanh_backend,
            attn_mask=ctx.attn_mask, document_ids=ctx.document_ids)
        return self.out_proj(y.reshape(b, t, self.attn_dim))
