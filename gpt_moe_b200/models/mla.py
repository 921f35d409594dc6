"""Multi-head latent attention (MLA).

One joint low-rank KV projection per token: `kv_down_proj` emits a latent of `kv_rank` plus one
shared RoPE key of `rope_dim`; `kv_up_proj` expands the normalised latent into per-head content
keys and values.  Queries are `content_dim + rope_dim` wide (optionally through a low-rank
`q_down_proj`/`q_norm`).  QK-norm is taken over the concatenated [content | rope] key and query;
softmax scale is (content+rope)^-0.5.  Parameter names and semantics follow the reference's MLA
experiment (`experiments/073-mla-current-kv768.patch:240-384`).

For generation the module keeps a latent cache (`MLACache`: latent, rope key and per-head key
gain per token) and decodes with absorbed weights: scores are taken directly against the latent
(`q_content @ W_k` folded into the query) and the context is produced in latent space and
expanded by `W_v` afterwards (same patch, lines 394-460).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
from torch import Tensor

from ..ops import api
from ..ops import reference as ref
from .attention import AttentionContext
from .linear import Linear
from .rotary import Rotary


@dataclass
class MLACache:
    latent: Tensor      # [B, S, kv_rank]
    rope: Tensor        # [B, S, rope_dim]
    key_gain: Tensor    # [B, S, n_kv_heads]  (QK-norm gain * clamped k_scale of the expanded key)
    length: int = 0


class MLAttention(nn.Module):
    def __init__(self, gpt_config, training_config, layer_idx: int = 0) -> None:
        super().__init__()
        self.n_heads = gpt_config.n_heads
        self.is_full_attention = layer_idx in gpt_config.full_attention_layers
        self.n_kv_heads = gpt_config.global_n_kv_heads if self.is_full_attention else gpt_config.n_kv_heads
        assert self.n_heads % self.n_kv_heads == 0
        self.group = self.n_heads // self.n_kv_heads
        self.q_rank, self.kv_rank = gpt_config.mla_q_rank, gpt_config.mla_kv_rank
        self.content_dim, self.rope_dim = gpt_config.mla_qk_content_dim, gpt_config.mla_qk_rope_dim
        self.value_dim = gpt_config.mla_value_dim
        self.head_size = self.content_dim + self.rope_dim
        self.attn_dim = self.n_heads * self.value_dim
        if self.q_rank < 0 or min(self.kv_rank, self.content_dim, self.value_dim) <= 0 or self.rope_dim < 0 or self.rope_dim % 2:
            raise ValueError("MLA needs q_rank >= 0, positive kv_rank/content/value dims and an even rope_dim >= 0")
        uses_rope = gpt_config.pos_encoding_type.lower() == "rope"
        if uses_rope != bool(self.rope_dim):
            raise ValueError("MLA: mla_qk_rope_dim must be > 0 with RoPE and 0 without")
        h = gpt_config.hidden_size
        if self.q_rank:
            self.q_down_proj = Linear(h, self.q_rank, role="q_proj", bias=gpt_config.use_bias)
            self.q_norm = nn.RMSNorm(self.q_rank, eps=gpt_config.mla_norm_eps)
        self.q_proj = Linear(self.q_rank or h, self.n_heads * self.head_size, role="q_proj", bias=gpt_config.use_bias)
        self.kv_down_proj = Linear(h, self.kv_rank + self.rope_dim, role="k_proj", bias=gpt_config.use_bias)
        self.kv_norm = nn.RMSNorm(self.kv_rank, eps=gpt_config.mla_norm_eps)
        self.kv_up_proj = Linear(self.kv_rank, self.n_kv_heads * (self.content_dim + self.value_dim),
                                 role="k_proj", bias=gpt_config.use_bias)
        self.out_proj = Linear(self.attn_dim, h, role="out_proj", bias=gpt_config.use_bias)
        theta = gpt_config.global_rope_theta if self.is_full_attention else gpt_config.rope_base_theta
        self.rotary = Rotary(self.rope_dim, theta, training_config.max_seq_len) if self.rope_dim else None
        self.use_qk_norm = gpt_config.use_qk_norm
        self.qk_norm_type = gpt_config.qk_norm_type
        self.qk_scale_min, self.qk_scale_max, self.qk_eps = gpt_config.qk_scale_min, gpt_config.qk_scale_max, gpt_config.qk_eps
        if self.use_qk_norm:
            self.q_scale = nn.Parameter(torch.full((1, self.n_heads, 1, 1), gpt_config.qk_scale_init))
            self.k_scale = nn.Parameter(torch.full((1, self.n_kv_heads, 1, 1), gpt_config.qk_scale_init))
        self.is_causal = gpt_config.is_causal
        self.use_flex_attention = gpt_config.use_flex_attention
        self.softmax_scale = self.head_size ** -0.5
        self.softcap = gpt_config.attn_logit_softcap if gpt_config.use_attn_logit_softcapping else 0.0
        self.tanh_backend = gpt_config.tanh_backend

    # ---- projections ---------------------------------------------------------------------------
    def _project(self, x: Tensor, start_pos: int = 0) -> Tuple[Tensor, Tensor, Tensor]:
        """-> query [B,T,H,content+rope] (rope part rotated), normalised latent [B,T,kv_rank], rotated rope key [B,T,1,rope]."""
        b, t, _ = x.shape
        query = x
        if self.q_rank:
            query = api.rms_norm(self.q_down_proj(query), self.q_norm.weight, self.q_norm.eps)
        query = self.q_proj(query).view(b, t, self.n_heads, self.head_size)
        compressed = self.kv_down_proj(x)
        latent, rope = compressed.split((self.kv_rank, self.rope_dim), dim=-1)
        latent = api.rms_norm(latent.contiguous(), self.kv_norm.weight, self.kv_norm.eps).to(compressed.dtype)
        rope = rope.reshape(b, t, 1, self.rope_dim)
        if self.rotary is not None:
            cos = self.rotary.cos_cached[start_pos:start_pos + t]
            sin = self.rotary.sin_cached[start_pos:start_pos + t]
            q_content, q_rope = query.split((self.content_dim, self.rope_dim), dim=-1)
            q_rope = ref.apply_rope(q_rope, cos, sin)
            rope = ref.apply_rope(rope, cos, sin)
            query = torch.cat((q_content, q_rope), dim=-1)
        return query, latent, rope

    def _gain(self, x: Tensor, scale: Tensor) -> Tensor:
        sq = x.pow(2)
        stat = sq.mean(dim=-1, keepdim=True) if self.qk_norm_type == "rms" else sq.sum(dim=-1, keepdim=True)
        gain = torch.rsqrt(stat + self.qk_eps).to(x.dtype)
        return gain * scale.clamp(self.qk_scale_min, self.qk_scale_max).reshape(1, 1, -1, 1).to(x.dtype)

    def _expand(self, query: Tensor, latent: Tensor, rope: Tensor, ctx: AttentionContext) -> Tuple[Tensor, Tensor]:
        b, t = latent.shape[:2]
        kv = self.kv_up_proj(latent).view(b, t, self.n_kv_heads, self.content_dim + self.value_dim)
        k_content, value = kv.split((self.content_dim, self.value_dim), dim=-1)
        key = torch.cat((k_content, rope.expand(-1, -1, self.n_kv_heads, -1)), dim=-1)
        if self.use_qk_norm:
            query = query * self._gain(query, self.q_scale)
            key_gain = self._gain(key, self.k_scale)
            key = key * key_gain
        else:
            key_gain = torch.ones_like(key[..., :1])
        out = api.attention(
            query, key, value.contiguous(), causal=self.is_causal,
            window=None if (self.is_full_attention or not self.use_flex_attention) else ctx.window,
            scale=self.softmax_scale, softcap_value=self.softcap, tanh_backend=self.tanh_backend,
            attn_mask=ctx.attn_mask, document_ids=ctx.document_ids)
        return out, key_gain

    def _fused_forward(self, x: Tensor, ctx: AttentionContext) -> Optional[Tensor]:
        """CUDA training path: the rotary rotation of the rope parts, the per-head QK-norm over the whole 128-wide head and the
        learned clamped scales run as ONE kernel over the packed [query heads | key heads] rows - the same kernel as for
        ordinary attention, given cos/sin tables that are the identity rotation on the content half of a head - followed by
        the 128/64-wide tcgen05 attention kernels.  Returns None when shapes or options need the general path."""
        b, t, _ = x.shape
        h, hk, d = self.n_heads, self.n_kv_heads, self.head_size
        if not (x.is_cuda and d == 128 and self.value_dim == 64 and self.rope_dim > 0 and self.rotary is not None and h + hk <= 64
                and t % 128 == 0 and self.is_causal and self.softcap == 0.0 and ctx.attn_mask is None and ctx.document_ids is None
                and self.q_proj.bias is None):
            return None
        from ..ops import cuda_ops
        query = x
        if self.q_rank:
            query = api.rms_norm(self.q_down_proj(query), self.q_norm.weight, self.q_norm.eps)
        query = self.q_proj(query).view(b, t, h, d)
        compressed = self.kv_down_proj(x)
        latent, rope = compressed.split((self.kv_rank, self.rope_dim), dim=-1)
        latent = api.rms_norm(latent.contiguous(), self.kv_norm.weight, self.kv_norm.eps).to(compressed.dtype)
        kv = self.kv_up_proj(latent).view(b, t, hk, self.content_dim + self.value_dim)
        k_content, value = kv.split((self.content_dim, self.value_dim), dim=-1)
        key = torch.cat((k_content, rope.reshape(b, t, 1, self.rope_dim).expand(-1, -1, hk, -1)), dim=-1)
        packed = torch.cat((query, key.to(query.dtype)), dim=2).to(torch.bfloat16)          # [B, T, H + Hkv, 128]: rows of heads
        if getattr(self, "_cos_padded", None) is None or self._cos_padded.device != x.device:
            # identity rotation (cos 1, sin 0) on the content pairs, the rotary tables on the rope pairs
            cos, sin = self.rotary.cos_cached.float(), self.rotary.sin_cached.float()
            pad = self.content_dim // 2
            self._cos_padded = torch.cat((torch.ones(cos.shape[0], pad, device=cos.device), cos), dim=1).contiguous()
            self._sin_padded = torch.cat((torch.zeros(sin.shape[0], pad, device=sin.device), sin), dim=1).contiguous()
        rotated = cuda_ops.rope_qk_norm_packed(
            packed.view(b * t, -1), self._cos_padded[:t], self._sin_padded[:t], self.q_scale if self.use_qk_norm else None,
            self.k_scale if self.use_qk_norm else None, t, h, hk, d, self.qk_eps, self.qk_norm_type == "rms",
            self.qk_scale_min, self.qk_scale_max).view(b, t, h + hk, d)
        out = api.attention(
            rotated[:, :, :h], rotated[:, :, h:], value.contiguous(), causal=True,
            window=None if (self.is_full_attention or not self.use_flex_attention) else ctx.window, scale=self.softmax_scale)
        return out

    def forward(self, x: Tensor, ctx: AttentionContext) -> Tensor:
        b, t, _ = x.shape
        out = self._fused_forward(x, ctx)
        if out is None:
            query, latent, rope = self._project(x)
            out, _ = self._expand(query, latent, rope, ctx)
        return self.out_proj(out.reshape(b, t, self.attn_dim))

    # ---- cached generation ---------------------------------------------------------------------
    def allocate_cache(self, batch_size: int, max_seq_len: int, *, device, dtype) -> MLACache:
        return MLACache(torch.zeros(batch_size, max_seq_len, self.kv_rank, device=device, dtype=dtype),
                        torch.zeros(batch_size, max_seq_len, self.rope_dim, device=device, dtype=dtype),
                        torch.zeros(batch_size, max_seq_len, self.n_kv_heads, device=device, dtype=dtype))

    @torch.no_grad()
    def forward_cached(self, x: Tensor, cache: MLACache, window: Optional[int] = None) -> Tensor:
        """Append x's tokens to the cache and attend over the whole cache with absorbed weights."""
        if self.training or not self.is_causal:
            raise ValueError("MLA cached forward requires causal attention in eval mode")
        b, t, _ = x.shape
        start, end = cache.length, cache.length + t
        if end > cache.latent.size(1) or b != cache.latent.size(0):
            raise ValueError("MLA cache capacity or batch size mismatch")
        query, latent, rope = self._project(x, start)
        cache.latent[:, start:end] = latent
        cache.rope[:, start:end] = rope[:, :, 0]
        w = self.kv_up_proj.weight.view(self.n_kv_heads, self.content_dim + self.value_dim, self.kv_rank)
        w_k, w_v = w[:, :self.content_dim].float(), w[:, self.content_dim:].float()
        # key gain of the new tokens needs their expanded keys (norm is over [content | rope])
        k_content = torch.einsum("btr,hdr->bthd", latent.float(), w_k)
        key = torch.cat((k_content, rope.float().expand(-1, -1, self.n_kv_heads, -1)), dim=-1)
        if self.use_qk_norm:
            cache.key_gain[:, start:end] = self._gain(key, self.k_scale)[..., 0].to(cache.key_gain.dtype)
            query = query * self._gain(query, self.q_scale)
        else:
            cache.key_gain[:, start:end] = 1.0
        cache.length = end
        q_content, q_rope = query.float().split((self.content_dim, self.rope_dim), dim=-1)
        q_content = q_content.view(b, t, self.n_kv_heads, self.group, self.content_dim)
        q_latent = torch.einsum("bthgd,hdr->bthgr", q_content, w_k).reshape(b, t, self.n_heads, self.kv_rank)
        context = api_mla_decode(q_latent, q_rope, cache.latent[:, :end], cache.rope[:, :end], cache.key_gain[:, :end],
                                 start, self.softmax_scale, self.softcap, self.tanh_backend,
                                 None if (self.is_full_attention or window is None) else int(window))
        context = context.view(b, t, self.n_kv_heads, self.group, self.kv_rank)
        out = torch.einsum("bthgr,hdr->bthgd", context, w_v).reshape(b, t, self.attn_dim)
        return self.out_proj(out.to(x.dtype))


def api_mla_decode(q_latent: Tensor, q_rope: Tensor, latent: Tensor, rope: Tensor, key_gain: Tensor,
                   start_pos: int, scale: float, softcap_value: float, tanh_backend: str,
                   window: Optional[int]) -> Tensor:
    """Absorbed-weight MLA decode: score = (q_latent . latent + q_rope . rope) * key_gain * scale over
    the cache, causal (query i sits at absolute position start_pos+i), optional window/softcap;
    returns the context in latent space [B,T,H,kv_rank] (fp32).
    Reference kernel: `experiments/073-mla-current-kv768.patch:456-673`."""
    b, t, h, r = q_latent.shape
    s_len = latent.shape[1]
    hkv = key_gain.shape[-1]
    g = h // hkv
    if (q_latent.is_cuda and latent.dtype == torch.bfloat16 and rope.dtype == torch.bfloat16 and key_gain.dtype == torch.bfloat16
            and (softcap_value <= 0.0 or tanh_backend == "exact")):
        # split-K decode kernel over the latent cache with a log-sum-exp merge (csrc/attention/mla_decode.cu)
        from ..ops import cuda_ops
        c = cuda_ops.ext()
        if c.mla_decode_ok(h, hkv, r, q_rope.shape[-1]):
            cuda_ops.count_path("mla_decode:kernel")
            return c.mla_decode(q_latent.float().contiguous(), q_rope.float().contiguous(), latent, rope, key_gain, int(start_pos),
                                float(scale), float(softcap_value), -1 if window is None else int(window))
        cuda_ops.count_path("mla_decode:torch")
    lat, rp = latent.float(), rope.float()
    score = torch.einsum("bthr,bsr->bhts", q_latent.float(), lat) + torch.einsum("bthd,bsd->bhts", q_rope.float(), rp)
    gain = key_gain.float().permute(0, 2, 1).repeat_interleave(g, dim=1)[:, :, None, :]
    score = ref.softcap(score * gain * scale, softcap_value, tanh_backend)
    qpos = torch.arange(start_pos, start_pos + t, device=score.device)[:, None]
    kpos = torch.arange(s_len, device=score.device)[None, :]
    keep = kpos <= qpos
    if window is not None:
        keep &= (qpos - kpos) <= window
    score = score.masked_fill(~keep, float("-inf"))
    return torch.einsum("bhts,bsr->bthr", torch.softmax(score, dim=-1), lat)
