"""Named presets for the benchmark configurations, and `key=value` overrides.

The reference has no CLI: variation is done by editing the dataclasses (`train.py:46,131`).  Here
the same two dataclasses are produced by `get_preset(name)` and then patched by
`apply_overrides(["model.n_layers=4", "training.seq_len_train=1024"])`.
"""
from __future__ import annotations

import ast
from dataclasses import fields
from typing import Iterable, Tuple

from .model import GPTConfig
from .training import TrainingConfig, default_linear_config
from ..schedules.token import custom_schedule


def _fixed_schedules(tc: TrainingConfig, batch: int, window: int) -> None:
    tc.batch_size_keys_schedule = {"fn": custom_schedule, "kwargs": {"values": [0]}}
    tc.batch_size_values_schedule = {"fn": custom_schedule, "kwargs": {"values": [batch]}}
    tc.swa_keys_schedule = {"fn": custom_schedule, "kwargs": {"values": [0]}}
    tc.swa_values_schedule = {"fn": custom_schedule, "kwargs": {"values": [window]}}


def _common_training(batch: int, seq: int, window: int, precision: str) -> TrainingConfig:
    tc = TrainingConfig(
        gpu_batch_size_train=batch, gpu_batch_size_val=batch, seq_len_train=seq, seq_len_val=seq,
        total_tokens_per_step_train=0, use_synthetic_data=True,
        linear_config=default_linear_config(precision), export_full_model_at_end=False,
        kernel_warmup_train_steps=1, val_tokens=2 * batch * seq,
    )
    _fixed_schedules(tc, batch, window)
    return tc


def tiny_cpu() -> Tuple[GPTConfig, TrainingConfig]:
    """2 layers, d_model 128, 4 heads x 32, 4 SwiGLU experts (hidden 512) top-1, full causal attention over 256 tokens, fp32."""
    gc = GPTConfig(n_layers=2, hidden_size=128, mlp_hidden_dim=512, use_tied_embeddings=False,
                   n_heads=4, n_kv_heads=4, attn_dim=128, rope_base_theta=10000,
                   activation="swiglu", use_fair_swiglu=False, num_experts=4, moe_top_k=1,
                   use_qk_debug_log=False)
    tc = _common_training(4, 256, 256, "default")
    tc.use_bf16_autocast = False
    tc.float32_matmul_precision = "highest"
    tc.max_tokens = 10 * 4 * 256
    return gc, tc


def _small_trunk(**kw) -> GPTConfig:
    base = dict(n_layers=12, hidden_size=768, use_tied_embeddings=False, n_heads=12, n_kv_heads=12,
                attn_dim=768, rope_base_theta=10000, activation="swiglu", use_fair_swiglu=False,
                use_qk_debug_log=False)
    base.update(kw)
    return GPTConfig(**base)


def small(precision: str = "default") -> Tuple[GPTConfig, TrainingConfig]:
    """GPT-MoE-small: 12L d768 12x64 heads, SWA 1024 over 2048 tokens, 8 SwiGLU experts (hidden 3072) top-1, micro-batch 16."""
    gc = _small_trunk(mlp_hidden_dim=3072, num_experts=8, moe_top_k=1)
    return gc, _common_training(16, 2048, 1024, precision)


def wide_ep(precision: str = "default") -> Tuple[GPTConfig, TrainingConfig]:
    """GPT-MoE-wide: small trunk, 32 SwiGLU experts (hidden 1536) top-2 renormalised gates, experts sharded over 8 ranks."""
    gc = _small_trunk(mlp_hidden_dim=1536, num_experts=32, moe_top_k=2)
    tc = _common_training(16, 2048, 1024, precision)
    tc.expert_parallel_size = 8
    return gc, tc


def mla(precision: str = "default") -> Tuple[GPTConfig, TrainingConfig]:
    """24L d1024 16 heads, MLA (kv rank 512, content 64 + rope 64, value 64), 64 routed SwiGLU experts (hidden 1024) top-1
    plus one shared SwiGLU expert (hidden 2048), experts sharded over 8 ranks, causal attention over 4096 tokens."""
    gc = GPTConfig(n_layers=24, hidden_size=1024, use_tied_embeddings=False, n_heads=16, n_kv_heads=16,
                   attn_dim=1024, rope_base_theta=10000, activation="swiglu", use_fair_swiglu=False,
                   mlp_hidden_dim=1024, num_experts=64, moe_top_k=1, moe_shared_expert_hidden_dim=2048,
                   use_mla=True, mla_kv_rank=512, mla_qk_content_dim=64, mla_qk_rope_dim=64,
                   mla_value_dim=64, use_qk_debug_log=False)
    tc = _common_training(8, 4096, 4096, precision)
    tc.expert_parallel_size = 8
    return gc, tc


PRESETS = {"tiny_cpu": tiny_cpu, "small": small, "wide_ep": wide_ep, "mla": mla}


def get_preset(name: str, **kwargs) -> Tuple[GPTConfig, TrainingConfig]:
    if name == "default":
        return GPTConfig(), TrainingConfig()
    return PRESETS[name](**kwargs)


def apply_overrides(gpt_config: GPTConfig, training_config: TrainingConfig, overrides: Iterable[str]) -> None:
    """Apply `model.<field>=<python literal>` / `training.<field>=<literal>` strings in place."""
    targets = {"model": gpt_config, "training": training_config}
    for item in overrides:
        key, _, raw = item.partition("=")
        scope, _, name = key.strip().partition(".")
        if scope not in targets or not name:
            raise ValueError(f"override must look like model.<field>=value or training.<field>=value: {item!r}")
        obj = targets[scope]
        if name not in {f.name for f in fields(obj)}:
            raise ValueError(f"unknown {scope} field: {name}")
        try:
            value = ast.literal_eval(raw)
        except (ValueError, SyntaxError):
            value = raw
        setattr(obj, name, value)
