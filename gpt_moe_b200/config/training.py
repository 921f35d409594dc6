"""Training configuration.

`TrainingConfig` keeps the reference's field names, defaults and `resolve(world_size)` contract
(`config/training.py:16-370`).  Differences by design:

* the tokenizer is resolved lazily (`get_tokenizer`) because the GPT-2 vocabulary may not be
  available offline; a byte-level fallback with the same `n_vocab` keeps everything runnable;
* precisions: `linear_config[phase][role]` accepts `"mxfp8"` (e4m3 with 32-element E8M0 block
  scales, the Blackwell-native recipe) next to `"default"` and `"fp8"`; backends are `"custom"`
  (this framework's kernels) and `"te"` (kept only as a recognised value: it maps to `"custom"`);
* new fields at the bottom control expert parallelism, sharded Muon and the fused collectives.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from datetime import datetime
from typing import Any, Dict, List, Optional, Tuple

import torch.nn as nn

from ..schedules.token import (add_schedule, custom_schedule, enforce_flex_block_constraints,
                               enforce_min_max_constraints, get_token_based_adamw_lr)

PHASES = ("training", "validation", "evaluation", "sampling")
ROLES = ("q_proj", "k_proj", "v_proj", "out_proj", "up_proj", "down_proj", "router", "lm_head")


def default_linear_config(training_precision: str = "default") -> Dict[str, Dict[str, Dict[str, str]]]:
    """All roles `default` outside training; in training the projection and expert roles use
    `training_precision` while the router and LM head stay in the surrounding (bf16/fp32) precision."""
    cfg: Dict[str, Dict[str, Dict[str, str]]] = {}
    for phase in PHASES:
        cfg[phase] = {}
        for role in ROLES:
            precision = "default"
            if phase == "training" and role not in ("router", "lm_head"):
                precision = training_precision
            cfg[phase][role] = {"precision": precision, "backend": "custom"}
    return cfg


_TIMESTAMP = datetime.now().strftime("%Y%m%d_%H%M%S")


@dataclass
class TrainingConfig:
    # parallelism: "ddp" (any world size, optionally with expert parallelism) or "pp" (2 stages)
    parallel_mode: str = "ddp"

    use_liger_loss: bool = False      # here: chunked fused LM-head + cross-entropy (never materialises logits)
    moe_load_balance_weight: float = 0.01

    # steps and tokens
    total_tokens_per_step_train: int = 2 ** 18
    gpu_batch_size_train: int = 8
    gpu_batch_size_val: int = 8
    seq_len_train: int = 8192
    seq_len_val: int = 8192
    max_tokens: int = 5 * 10 ** 9

    flex_block_size: int = 128
    enforce_even_blocks: bool = False
    batch_size_keys_schedule: Dict[str, Any] = field(default_factory=lambda: {
        "fn": custom_schedule, "kwargs": {"values": [0, 78_643_200]}})
    batch_size_values_schedule: Dict[str, Any] = field(default_factory=lambda: {
        "fn": custom_schedule, "kwargs": {"values": [4, 8]}})
    swa_keys_schedule: Dict[str, Any] = field(default_factory=lambda: {
        "fn": add_schedule, "kwargs": {"start": 32_768_000, "increment": 200 * 262_144, "count": 11}})
    swa_values_schedule: Dict[str, Any] = field(default_factory=lambda: {
        "fn": add_schedule, "kwargs": {"start": 128, "increment": 128, "count": 11}})
    # filled by resolve()
    batch_size_schedule_keys: List[int] = field(init=False, default_factory=list)
    batch_size_schedule_values: List[int] = field(init=False, default_factory=list)
    swa_schedule_keys: List[int] = field(init=False, default_factory=list)
    swa_schedule_values: List[int] = field(init=False, default_factory=list)
    swa_initial_window_size: int = field(init=False, default=0)
    swa_final_window_size: int = field(init=False, default=0)
    max_seq_len: int = field(init=False, default=0)
    max_train_steps: int = field(init=False, default=0)

    tokenizer: Any = None             # resolved lazily, see get_tokenizer()
    tokenizer_name: str = "gpt2"

    # optimizers
    adamw_betas: Tuple[float, float] = (0.9, 0.95)
    adamw_eps: float = 1e-8
    adamw_max_lr: float = 5e-3
    lr_warmup_tokens: int = 0
    lr_warmup_and_cosine_tokens: int = 600 * 10 ** 6
    adamw_weight_decay: float = 0.01
    adamw_hard_min_lr: float = 7e-4
    optimizer_type: str = "muon"      # "muon" (+adamw) or anything else for adamw only
    muon_lr_scale: float = 0.15
    muon_backend: str = "polarexpress"  # svd | newtonschulz5 | polarexpress
    muon_backend_steps: int = 5
    muon_momentum: float = 0.95
    muon_use_nesterov: bool = True
    total_decay_tokens: int = field(init=False, default=0)
    lr_schedule: List[Dict[str, Any]] = field(default_factory=list)

    # checkpointing
    enable_checkpointing: bool = False
    checkpoint_interval: int = -1
    checkpoint_best_improvement_interval: int = -1
    max_checkpoints_to_keep: int = 3
    export_full_model_at_end: bool = True
    full_model_export_interval: int = -1
    resume_from_checkpoint: bool = False
    resume_checkpoint_path: str = ""
    resume_state_dict_path: str = ""
    resume_timestamp: str = ""
    hf_user: Any = field(default_factory=lambda: os.environ.get("hf_user"))
    hf_token: Any = field(default_factory=lambda: os.environ.get("hf_token"))
    timestamp: str = ""
    checkpoint_dir: str = ""
    model_export_dir: str = ""
    hub_repo_id: str = ""

    # logging
    config_and_log_dir: str = ""
    log_filename: str = ""
    config_filename: str = ""

    # data
    data_path: str = "./data/edu_fineweb10B"
    data_uses_padding: bool = False

    # validation
    val_target: float = 3.28
    val_tokens: int = 5 * 2 ** 21
    shuffle_val_tokens: bool = False
    val_interval: int = 25
    train_val_margin: float = -9.0

    # sampling
    sample_interval: int = 25
    run_sampling: bool = False
    sample_sequences: List[str] = field(default_factory=lambda: [
        "The universe has always been",
        "Who am I? I am a language model",
        "Artificial General Intelligence is",
        "Artificial General Intelligence is not",
        "2+2 is",
        "The quick brown fox jumps",
        "Earth is",
        "Could you tell me what time it is?",
    ])

    hellaswag_interval: int = 50
    run_benchmarks: bool = False

    run_gsm8k: bool = False
    gsm8k_interval: int = -1
    gsm8k_max_examples: int = -1
    gsm8k_num_shots: int = 8
    gsm8k_examples_per_batch: int = 4
    gsm8k_max_new_tokens: int = 512

    base_seed: int = 1337
    kernel_warmup_train_steps: int = 2
    use_activation_checkpointing: bool = False
    activation_offload_layers: int = 0
    activation_offload_min_bytes: int = 1024 * 1024

    # Kept for config-surface parity.  This framework has no tracing compiler: the fields select
    # whether launch-bound regions (optimizer step) are replayed from CUDA graphs
    # ("max-autotune"/"reduce-overhead") or launched eagerly ("*-no-cudagraphs"/"default").
    torch_compile_mode_no_grad_accum: str = "max-autotune"
    torch_compile_mode_grad_accum: str = "max-autotune-no-cudagraphs"
    torch_compile_fullgraph: bool = True
    torch_compile_dynamic: bool = False

    linear_config: Dict[str, Dict[str, Dict[str, str]]] = field(default_factory=default_linear_config)

    keep_fp32_loss: bool = True
    use_bf16_adamw_moments: bool = False
    use_all_bf16_and_null_ctx: bool = False
    use_bf16_weights_params_or_scales: bool = False
    bf16_weights_params_and_scales: Dict[str, Any] = field(default_factory=lambda: {
        "nn.Linear": nn.Linear, "nn.Embedding": nn.Embedding})
    float32_matmul_precision: str = "high"
    use_bf16_autocast: bool = True
    keep_1d_weights_params_and_scales_in_fp32: bool = False
    cast_activations_to_weight_dtype_if_no_autocast: bool = False

    # filled by resolve()
    total_tokens_per_mini_step_train: int = field(init=False, default=0)
    grad_accum_mini_steps: int = field(init=False, default=0)
    total_tokens_per_step_val: int = field(init=False, default=0)
    val_steps: int = field(init=False, default=0)
    torch_compile_mode: str = field(init=False, default="")

    # ---- new capabilities ---------------------------------------------------------------------
    expert_parallel_size: int = 1     # experts are sharded over this many ranks (must divide world size and num_experts)
    shard_muon: bool = True           # each rank orthogonalises only the matrices it owns, then all-gathers
    grad_reduce_dtype: str = "fp32"   # wire dtype of the Muon gradient reduction: "fp32" (the reference's DDP precision) or "bf16"
                                      # (peers read a bf16 shadow of the gradient buffer, the owner still sums in fp32)
    grad_bucket_mb: int = 64          # flat gradient bucket size
    use_fused_collectives: bool = True  # peer-memory kernels; False = NCCL calls (the measured baseline)
    use_cuda_graphs: bool = True        # fused engine: forward+backward of a training step is captured once per (shape, window) and replayed
    nvtx_ranges: bool = False           # NVTX ranges around the phases of a training step (forward+backward per micro-step, optimizer)
    overlap_grad_reduce: Optional[bool] = None   # fused engine: a block's gradient reduce (+ momentum, pack) runs on a second stream beside
                                        # the backward of the earlier blocks; orthogonalisation and the weight push follow the backward
                                        # pass.  None = on from 4 ranks up (with two the hidden transfer is smaller than the cost)
    allow_nccl_fallback: bool = False   # fused engine requested but symmetric memory unavailable: fall back to NCCL instead of raising
    ep_capacity_factor: float = 0.0     # fused expert parallelism: receive buffers hold this many times a rank's own slots (0 = worst case)
    step_deadline_s: float = 0.0      # >0 arms the host watchdog: abort the job if a step exceeds it
    use_synthetic_data: bool = False  # uniform random token ids from `base_seed` instead of .npy shards

    def __post_init__(self) -> None:
        if not self.timestamp:
            self.timestamp = self.resume_timestamp if self.resume_from_checkpoint else _TIMESTAMP
        if not self.checkpoint_dir:
            self.checkpoint_dir = f"./checkpoints/{self.timestamp}"
        if not self.model_export_dir:
            self.model_export_dir = f"./model_exports/{self.timestamp}"
        if not self.hub_repo_id:
            self.hub_repo_id = f"{self.hf_user}/nanogpt_{self.timestamp}"
        if not self.config_and_log_dir:
            self.config_and_log_dir = f"./configs_and_logs/{self.timestamp}"
        if not self.log_filename:
            self.log_filename = os.path.join(self.config_and_log_dir, "log.txt")
        if not self.config_filename:
            self.config_filename = os.path.join(self.config_and_log_dir, "config.txt")
        self.max_seq_len = max(self.seq_len_train, self.seq_len_val)
        self.max_train_steps = self.max_tokens // max(1, self.total_tokens_per_step_train)
        self.total_decay_tokens = self.lr_warmup_and_cosine_tokens - self.lr_warmup_tokens

    # -------------------------------------------------------------------------------------------
    def resolve(self, world_size: int) -> None:
        """Derive step counts and materialise the schedules for a data-parallel size.

        Same derivations as the reference `config/training.py:287-370`.
        """
        if self.use_all_bf16_and_null_ctx:
            self.use_bf16_autocast = False
            self.bf16_weights_params_and_scales = {"all": object}
        if self.optimizer_type == "muon" and self.muon_backend == "polarexpress":
            assert self.muon_backend_steps == 5, (
                "Polar Express uses five pre-computed coefficient triples; "
                f"muon_backend_steps must be 5 (got {self.muon_backend_steps})")
        self.max_seq_len = max(self.seq_len_train, self.seq_len_val)
        self.total_tokens_per_mini_step_train = world_size * self.gpu_batch_size_train * self.seq_len_train
        if self.total_tokens_per_step_train <= 0:     # "one mini-step per step at any world size" (weak scaling)
            self.total_tokens_per_step_train = self.total_tokens_per_mini_step_train
        assert self.total_tokens_per_step_train % self.total_tokens_per_mini_step_train == 0, \
            "total_tokens_per_step_train must be a multiple of the tokens in one mini-step"
        self.grad_accum_mini_steps = self.total_tokens_per_step_train // self.total_tokens_per_mini_step_train
        self.max_train_steps = self.max_tokens // self.total_tokens_per_step_train
        self.total_tokens_per_step_val = world_size * self.gpu_batch_size_val * self.seq_len_val
        self.val_steps = math.ceil(self.val_tokens / self.total_tokens_per_step_val)
        self.total_decay_tokens = self.lr_warmup_and_cosine_tokens - self.lr_warmup_tokens
        self.torch_compile_mode = (self.torch_compile_mode_no_grad_accum if self.grad_accum_mini_steps == 1
                                   else self.torch_compile_mode_grad_accum)

        def materialise(spec: Dict[str, Any]) -> List[int]:
            return enforce_min_max_constraints(spec["fn"](**spec["kwargs"]), spec.get("min"), spec.get("max"))

        self.batch_size_keys_schedule["max"] = self.max_tokens
        self.batch_size_schedule_keys = materialise(self.batch_size_keys_schedule)
        self.batch_size_schedule_values = materialise(self.batch_size_values_schedule)
        self.swa_keys_schedule["max"] = self.max_tokens
        self.swa_schedule_keys = materialise(self.swa_keys_schedule)
        self.swa_schedule_values = [
            enforce_flex_block_constraints(v, self.flex_block_size, self.enforce_even_blocks)
            for v in materialise(self.swa_values_schedule)]
        self.swa_initial_window_size = self.swa_schedule_values[0]
        self.swa_final_window_size = self.swa_schedule_values[-1]

        self.lr_schedule = [{
            "start": 0, "end": self.max_tokens, "fn": get_token_based_adamw_lr,
            "kwargs": {
                "lr_warmup_tokens": self.lr_warmup_tokens,
                "lr_warmup_and_cosine_tokens": self.lr_warmup_and_cosine_tokens,
                "total_decay_tokens": self.total_decay_tokens,
                "adamw_max_lr": self.adamw_max_lr,
                "adamw_hard_min_lr": self.adamw_hard_min_lr,
            },
        }]

    def get_tokenizer(self):
        if self.tokenizer is None:
            from ..tokenizer import load_tokenizer
            self.tokenizer = load_tokenizer(self.tokenizer_name)
        return self.tokenizer


RESUME_TRAINING_FIELDS = (
    "parallel_mode", "total_tokens_per_step_train", "gpu_batch_size_train", "seq_len_train",
    "grad_accum_mini_steps", "batch_size_schedule_keys", "batch_size_schedule_values",
    "swa_schedule_keys", "swa_schedule_values", "max_seq_len", "flex_block_size",
    "swa_initial_window_size", "data_path", "data_uses_padding", "base_seed", "optimizer_type",
    "adamw_betas", "adamw_eps", "adamw_weight_decay", "muon_lr_scale", "muon_backend",
    "muon_backend_steps", "muon_momentum", "muon_use_nesterov", "moe_load_balance_weight",
    "use_bf16_autocast", "use_all_bf16_and_null_ctx", "use_bf16_weights_params_or_scales",
    "use_bf16_adamw_moments", "keep_1d_weights_params_and_scales_in_fp32", "keep_fp32_loss",
    "cast_activations_to_weight_dtype_if_no_autocast", "use_liger_loss", "linear_config",
)


def build_resume_config(gpt_config, training_config: TrainingConfig) -> Dict[str, Any]:
    """The dictionary whose equality decides whether a checkpoint may be resumed.

    Same three sections and key set as the reference builds inline (`train.py:131-158`), so a
    training-state file written by either program compares equal under the other when the shared
    fields agree.  Fields that only this framework has are appended under `"b200"`.
    """
    from dataclasses import asdict
    return {
        "model": asdict(gpt_config),
        "training": {name: getattr(training_config, name) for name in RESUME_TRAINING_FIELDS},
        "bf16_weights_params_and_scales": {
            name: f"{value.__module__}.{value.__qualname__}"
            for name, value in training_config.bf16_weights_params_and_scales.items()},
        "lr_schedule": [
            {"start": s["start"], "end": s["end"], "fn": s["fn"].__name__, "kwargs": s["kwargs"]}
            for s in training_config.lr_schedule],
        "b200": {"expert_parallel_size": training_config.expert_parallel_size},
    }
