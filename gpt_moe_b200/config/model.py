"""Model architecture configuration.

`GPTConfig` keeps every field name and default of the reference dataclass
(`config/model.py:8-94`) so that configs, `resume_config` dictionaries and exported
`*_config.json` files stay interchangeable.  Fields below the "new capabilities" marker do not
exist in the reference; their defaults reproduce reference behaviour.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List


@dataclass
class GPTConfig:
    # trunk
    n_layers: int = 8
    hidden_size: int = 1024
    use_bias: bool = False
    mlp_hidden_dim: int = 2048
    use_tied_embeddings: bool = True
    norm_type: str = "rms"            # "rms"; anything else selects LayerNorm
    is_causal: bool = True

    # residual weighting: x = alpha*x + beta*f(norm(x)); alpha/beta learned scalars when enabled
    use_weighted_residual_path: bool = False
    weighted_residual_path_init: float = 1.0
    use_weighted_main_path: bool = True
    weighted_main_path_init: float = 0.0

    # vocabulary
    vocab_size: int = 50304
    pad_token_id: int = 50257
    eos_token_id: int = 50256

    # local (sliding-window) attention; n_kv_heads < n_heads gives GQA, ==1 gives MQA
    n_heads: int = 16
    n_kv_heads: int = 16
    attn_dim: int = 1024
    use_flex_attention: bool = True   # True: block-sparse masked attention (SWA/doc/softcap allowed); False: plain SDPA semantics
    use_doc_masking: bool = False
    use_attn_logit_softcapping: bool = False
    attn_logit_softcap: float = 15.0
    tanh_backend: str = "ptx"         # "clamp" | "ptx" | "rational" | "exact"

    use_qk_norm: bool = True
    qk_norm_type: str = "rms"         # "rms"; anything else selects L2
    qk_scale_init: float = 1.0
    qk_scale_min: float = float("-inf")
    qk_scale_max: float = 5.0
    qk_eps: float = 1e-6
    use_qk_debug_log: bool = True

    # positions
    pos_encoding_type: str = "rope"   # "rope" | "nope" | anything else = learned absolute
    rope_base_theta: int = 500_000

    # per-layer full (global) attention overrides
    full_attention_layers: List[int] = field(default_factory=list)
    global_attn_dim: int = 2048
    global_n_kv_heads: int = 4
    global_rope_theta: int = 500_000

    # feed-forward
    activation: str = "relu2"         # gelu | relu | relu2 | silu | swiglu
    use_fair_swiglu: bool = True

    # mixture of experts
    use_moe: bool = True
    num_experts: int = 16
    moe_top_k: int = 1
    moe_full_softmax_gating: bool = False

    # ---- new capabilities (absent from the reference's live tree) --------------------------
    # multi-head latent attention (reference: experiments/073-mla-current-kv768.patch:8-16)
    use_mla: bool = False
    mla_q_rank: int = 0               # 0 = full-rank query projection
    mla_kv_rank: int = 512
    mla_qk_content_dim: int = 64
    mla_qk_rope_dim: int = 64
    mla_value_dim: int = 64
    mla_norm_eps: float = 1e-6
    mla_recompute_attention: bool = False
    # shared (always-on) expert beside the routed ones; 0 disables
    moe_shared_expert_hidden_dim: int = 0

    @property
    def head_size(self) -> int:
        return self.attn_dim // self.n_heads
