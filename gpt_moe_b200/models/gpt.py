"""The GPT-MoE language model.

Same constructor, forward signature, state-dict keys and optimizer split as the reference
`GPT` (`model/gpt.py:22-842`):

* `GPT(gpt_config, training_config, stage_index=None)`; stage 0/1 keep half of the blocks for the
  two-stage pipeline.
* `forward(indices, targets, attn_mask, ignore_doc_mask, document_ids, previous_stage_balance_loss)`
  returns `(loss, token_loss, balance_term)` in training, `loss` in eval with targets, logits
  without targets.
* `sliding_window_size` is a non-persistent 0-dim int32 buffer: the window schedule changes it
  with `fill_` and the attention kernel reads it on the device, so nothing is re-launched or
  re-built when the window grows.

Masking differs by design: the reference builds FlexAttention block masks
(`model/gpt.py:311-687`); here causal / window / padding / document constraints are evaluated
token-exactly inside the attention op (window inclusive: q - k <= W).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple, Union

import torch
import torch.nn as nn
from torch import Tensor
from torch.utils.checkpoint import checkpoint

from ..config.training import PHASES, ROLES
from ..ops import api
from .attention import AttentionContext
from .block import Block, apply_norm, make_norm
from .linear import Linear


def validate_linear_config(linear_config, use_moe: bool) -> List[str]:
    """Reject unsupported precision/backend combinations with the role named (reference `model/gpt.py:68-86`).

    Backends: "custom" is this framework's MXFP8 path.  "te" names the reference's Transformer Engine block-scaled linear
    (`model/linear/fp8/transformer_engine.py:10-34`: e4m3 with 1x128 activation and 128x128 weight blocks); Transformer Engine
    is not part of this framework, so an fp8 role with backend "te" runs on the same MXFP8 kernels (32-element E8M0 blocks:
    finer scaling than TE's recipe, same operand format) — the returned list names those `phase.role` entries so the caller
    can say so in the log instead of switching silently."""
    remapped: List[str] = []
    for phase in PHASES:
        for role in ROLES:
            policy = linear_config[phase][role]
            precision, backend = policy["precision"], policy["backend"]
            if precision not in ("default", "fp8", "mxfp8"):
                raise ValueError(f"unsupported linear precision for {phase}.{role}: {precision}")
            if backend not in ("custom", "te"):
                raise ValueError(f"unsupported linear backend for {phase}.{role}: {backend}")
            if precision != "default" and role == "router":
                raise ValueError(f"{phase}.{role}: the router stays in fp32/bf16; use precision='default'")
            if precision != "default" and backend == "te":
                remapped.append(f"{phase}.{role}")
    return remapped


class GPT(nn.Module):
    def __init__(self, gpt_config, training_config, stage_index: Optional[int] = None,
                 ep_rank: int = 0, ep_size: int = 1) -> None:
        super().__init__()
        self.gpt_config = gpt_config
        self.stage_index = stage_index
        self.max_seq_len = training_config.max_seq_len
        self.pad_token_id = gpt_config.pad_token_id
        self.pos_encoding_type = gpt_config.pos_encoding_type.lower()
        self.optimizer_type = training_config.optimizer_type.lower()
        self.use_activation_checkpointing = training_config.use_activation_checkpointing
        self.muon_lr_scale = training_config.muon_lr_scale
        self.muon_backend = training_config.muon_backend
        self.muon_backend_steps = training_config.muon_backend_steps
        self.muon_momentum = training_config.muon_momentum
        self.muon_use_nesterov = training_config.muon_use_nesterov
        self.use_qk_norm = gpt_config.use_qk_norm
        self.use_qk_debug_log = gpt_config.use_qk_debug_log
        self.is_causal = gpt_config.is_causal
        self.use_flex_attention = gpt_config.use_flex_attention
        self.use_doc_masking = gpt_config.use_doc_masking
        self.data_uses_padding = training_config.data_uses_padding
        self.keep_fp32_loss = training_config.keep_fp32_loss
        self.use_liger_loss = training_config.use_liger_loss
        self.linear_config = training_config.linear_config
        self.te_roles_on_mxfp8 = validate_linear_config(self.linear_config, gpt_config.use_moe)
        self.moe_load_balance_weight = training_config.moe_load_balance_weight
        self.num_moe_layers = gpt_config.n_layers if gpt_config.use_moe else 0

        swa_values = training_config.swa_schedule_values or [training_config.max_seq_len]
        if gpt_config.use_doc_masking or gpt_config.use_attn_logit_softcapping or min(swa_values) < training_config.max_seq_len:
            assert self.use_flex_attention, "document masking / sliding window / attention soft-capping require use_flex_attention=True"
        self.initial_sliding_window_size = swa_values[0]
        self.register_buffer("sliding_window_size",
                             torch.tensor(self.initial_sliding_window_size, dtype=torch.int32), persistent=False)

        for idx in gpt_config.full_attention_layers:
            assert 0 <= idx < gpt_config.n_layers, f"full_attention_layers index {idx} out of range"
        self.layer_is_full_attention = [i in set(gpt_config.full_attention_layers) for i in range(gpt_config.n_layers)]

        modules = dict(wte=nn.Embedding(gpt_config.vocab_size, gpt_config.hidden_size))
        if self.pos_encoding_type not in ("rope", "nope"):
            modules["wpe"] = nn.Embedding(training_config.max_seq_len, gpt_config.hidden_size)
        modules["h"] = nn.ModuleList([Block(gpt_config, training_config, layer_idx=i, ep_rank=ep_rank, ep_size=ep_size)
                                      for i in range(gpt_config.n_layers)])
        modules["ln_f"] = make_norm(gpt_config)
        self.transformer = nn.ModuleDict(modules)
        self.lm_head = Linear(gpt_config.hidden_size, gpt_config.vocab_size, role="lm_head", bias=False)

        self.use_tied_embeddings = gpt_config.use_tied_embeddings
        if self.use_tied_embeddings:
            self.transformer.wte.weight = self.lm_head.weight
        self.apply(self._init_weights)
        if ep_size > 1:
            for block in self.transformer.h:
                if block.use_moe:
                    block.mlp.keep_local_experts()

        if stage_index is not None:
            assert not self.use_tied_embeddings, "pipeline parallelism requires untied embeddings"
            split = gpt_config.n_layers // 2
            assert 0 < split < gpt_config.n_layers, "pipeline parallelism requires at least two blocks"
            if stage_index == 0:
                self.transformer.h = self.transformer.h[:split]
                self.layer_is_full_attention = self.layer_is_full_attention[:split]
                del self.transformer["ln_f"]
                del self.lm_head
            else:
                self.transformer.h = self.transformer.h[split:]
                self.layer_is_full_attention = self.layer_is_full_attention[split:]
                del self.transformer["wte"]
                if "wpe" in self.transformer:
                    del self.transformer["wpe"]

        self.activation_offloader = None
        if not 0 <= training_config.activation_offload_layers <= len(self.transformer.h):
            raise ValueError("activation_offload_layers must be between 0 and the number of blocks on this GPU")
        if training_config.activation_offload_layers:
            from ..runtime.activation_offloading import ActivationOffloading
            if training_config.activation_offload_min_bytes < 0:
                raise ValueError("activation_offload_min_bytes must be non-negative")
            self.activation_offloader = ActivationOffloading(
                training_config.activation_offload_layers, training_config.activation_offload_min_bytes)

        self._linear_modules = tuple(m for m in self.modules() if isinstance(m, Linear))
        self.precision_phase = None
        self.set_precision_phase("training")

    def set_sliding_window(self, window: int) -> None:
        """Update the device-resident window and remember the host value (ops that need a host integer read
        it from the buffer's `host_value` attribute instead of synchronising)."""
        self.sliding_window_size.fill_(int(window))
        self.sliding_window_size.host_value = int(window)

    # ---- precision phases ---------------------------------------------------------------------
    def set_precision_phase(self, phase: str) -> None:
        if phase == self.precision_phase:
            return
        self.clear_fp8_weights()
        policy = self.linear_config[phase]
        for module in self._linear_modules:
            module.precision = policy[module.role]["precision"]
            module.backend = policy[module.role]["backend"]
        self.precision_phase = phase

    def prepare_fp8_weights(self) -> None:
        """Quantise the MXFP8 weights once, ahead of the micro-steps of a gradient-accumulation step (reference
        `train.py:379-380`).  On the GPU the quantised copies (row-wise for the forward GEMM, transposed for the
        input-gradient GEMM) live in `ops.cuda_ops`' parameter-epoch cache: this fills it, later uses hit it until an
        optimizer step or `clear_fp8_weights` invalidates it.  Nothing to do on the CPU path, which quantises inline."""
        if not any(p.is_cuda for p in self.parameters()):
            return
        from ..ops import mxfp8
        for block in self.transformer.h:
            mxfp8.prepare_block_weights(block)

    def clear_fp8_weights(self) -> None:
        """Drop the quantised weight copies (before an optimizer step, on a phase change, at exit: reference
        `train.py:488, 755`, `model/gpt.py:198`)."""
        if any(p.is_cuda for p in self.parameters()):
            from ..ops import mxfp8
            mxfp8.clear_quantized_weights()

    def _init_weights(self, module: nn.Module) -> None:
        if isinstance(module, nn.Linear):
            torch.nn.init.normal_(module.weight, mean=0.0, std=0.02)
            if module.bias is not None:
                torch.nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            torch.nn.init.normal_(module.weight, mean=0.0, std=0.02)

    # ---- optimizers ---------------------------------------------------------------------------
    def optimizer_param_groups(self) -> Dict[str, List[Tuple[str, nn.Parameter]]]:
        """Split trainable parameters: Muon takes every 2-D matrix whose name has no wte/wpe/lm_head
        (router included); AdamW-decay takes the other >=2-D tensors; AdamW-no-decay the <2-D ones
        (reference `model/gpt.py:253-267`)."""
        named = [(n, p) for n, p in self.named_parameters() if p.requires_grad]
        muon = []
        if self.optimizer_type == "muon":
            muon = [(n, p) for n, p in named if p.dim() == 2 and not any(t in n for t in ("wte", "wpe", "lm_head"))]
        muon_names = {n for n, _ in muon}
        rest = [(n, p) for n, p in named if n not in muon_names]
        return {"muon": muon,
                "adamw_decay": [(n, p) for n, p in rest if p.dim() >= 2],
                "adamw_nodecay": [(n, p) for n, p in rest if p.dim() < 2]}

    def configure_optimizers(self, lr: float, adamw_betas: Tuple[float, float], adamw_eps: float,
                             adamw_weight_decay: float, device_type: str, *, muon_class=None,
                             master_process: bool = False, log_buffer: Optional[List[str]] = None,
                             ) -> Dict[str, torch.optim.Optimizer]:
        from ..optim.adamw import AdamW
        from ..optim.muon import Muon
        muon_class = muon_class or Muon
        groups = self.optimizer_param_groups()
        if master_process:
            msgs = [
                f"num decayed parameter tensors (AdamW): {len(groups['adamw_decay'])}, with {sum(p.numel() for _, p in groups['adamw_decay']):,} parameters",
                f"num non-decayed parameter tensors (AdamW): {len(groups['adamw_nodecay'])}, with {sum(p.numel() for _, p in groups['adamw_nodecay']):,} parameters",
            ]
            if self.optimizer_type == "muon":
                msgs.append(f"num Muon parameter tensors: {len(groups['muon'])}, with {sum(p.numel() for _, p in groups['muon']):,} parameters")
            for m in msgs:
                print(m)
                if log_buffer is not None:
                    log_buffer.append(m)
        adamw = AdamW([
            {"params": [p for _, p in groups["adamw_decay"]], "weight_decay": adamw_weight_decay},
            {"params": [p for _, p in groups["adamw_nodecay"]], "weight_decay": 0.0},
        ], lr=lr, betas=adamw_betas, eps=adamw_eps)
        if self.optimizer_type != "muon":
            return {"adamw": adamw}
        muon = muon_class([p for _, p in groups["muon"]], lr=lr * self.muon_lr_scale, momentum=self.muon_momentum,
                          nesterov=self.muon_use_nesterov, backend=self.muon_backend, backend_steps=self.muon_backend_steps)
        return {"adamw": adamw, "muon": muon}

    # ---- forward ------------------------------------------------------------------------------
    def _attention_context(self, attn_mask: Optional[Tensor], document_ids: Optional[Tensor],
                           ignore_doc_mask: bool, batch: int, seq_len: int, device) -> AttentionContext:
        if attn_mask is not None:
            if attn_mask.dim() != 2 or tuple(attn_mask.shape) != (batch, seq_len):
                raise ValueError(f"attn_mask must be [gpu_batch_size, seq_len] = [{batch}, {seq_len}], got {list(attn_mask.shape)}")
            attn_mask = attn_mask.to(device=device, dtype=torch.bool, non_blocking=True)
        docs = document_ids if (self.use_doc_masking and not ignore_doc_mask) else None
        window = self.sliding_window_size if self.use_flex_attention else None
        return AttentionContext(window, attn_mask, docs)

    def forward(self, indices: Tensor, targets: Optional[Tensor] = None, attn_mask: Optional[Tensor] = None,
                ignore_doc_mask: bool = False, document_ids: Optional[Tensor] = None,
                previous_stage_balance_loss: Optional[Tensor] = None,
                ) -> Union[Tensor, Tuple[Tensor, Optional[Tensor]], Tuple[Tensor, Tensor, Tensor]]:
        batch, seq_len = indices.shape[:2]
        if self.stage_index != 1:
            x = self.transformer.wte(indices)
            if "wpe" in self.transformer:
                x = x + self.transformer.wpe(torch.arange(seq_len, dtype=torch.long, device=indices.device))
        else:
            x = indices
        ctx = self._attention_context(attn_mask, document_ids, ignore_doc_mask, batch, seq_len, x.device)

        balance_loss = None
        grad_mode = self.training and torch.is_grad_enabled()
        blocks = self.transformer.h
        chain = (self.stage_index is None and isinstance(self.transformer.ln_f, nn.RMSNorm) and len(blocks) > 0
                 and not (grad_mode and (self.use_activation_checkpointing or self.activation_offloader is not None)))
        if chain:
            # residual update + following RMSNorm as one op per link (see Block.forward_prenormed)
            h = apply_norm(blocks[0].ln_1, x)
            hook = getattr(self, "block_grad_hook", None) if grad_mode else None
            for i, block in enumerate(blocks):
                if hook is not None and h.requires_grad:
                    # the gradient of a block's normalised input is the last thing its backward produces
                    h.register_hook(lambda grad, layer=i, fn=hook: fn(layer))
                next_norm = blocks[i + 1].ln_1 if i + 1 < len(blocks) else self.transformer.ln_f
                next_q = getattr(blocks[i + 1].attn, "q_proj", None) if i + 1 < len(blocks) else None
                next_mxfp8 = next_q is not None and next_q.precision in ("mxfp8", "fp8") and hasattr(blocks[i + 1].attn, "k_proj")
                x, h, block_balance = block.forward_prenormed(x, h, ctx, next_norm, next_mxfp8)
                if block_balance is not None:
                    balance_loss = block_balance if balance_loss is None else balance_loss + block_balance
            x = h
        elif self.activation_offloader is not None and grad_mode:
            x, balance_loss = self.activation_offloader.run(self.transformer.h, x, ctx)
        else:
            for block in self.transformer.h:
                if self.use_activation_checkpointing and grad_mode:
                    x, block_balance = checkpoint(block, x, ctx, use_reentrant=False)
                else:
                    x, block_balance = block(x, ctx)
                if block_balance is not None:
                    balance_loss = block_balance if balance_loss is None else balance_loss + block_balance
        if self.stage_index == 0:
            return (x, balance_loss) if balance_loss is not None else x

        if not chain:
            x = apply_norm(self.transformer.ln_f, x)
        ignore_index = self.pad_token_id if self.data_uses_padding else -100
        logits = None
        if targets is not None and (self.use_liger_loss or (x.is_cuda and self.training)):
            # fused LM head + streaming fp32 cross-entropy: logits are never materialised
            loss = api.linear_cross_entropy(x.reshape(-1, x.size(-1)), self.lm_head.weight, targets.reshape(-1), ignore_index)
        else:
            logits = self.lm_head(x)
            loss = api.cross_entropy(logits.view(-1, logits.size(-1)), targets.reshape(-1), ignore_index) if targets is not None else None

        if previous_stage_balance_loss is not None:
            balance_loss = previous_stage_balance_loss if balance_loss is None else balance_loss + previous_stage_balance_loss
        if targets is not None:
            token_loss = loss
            balance_term = loss.new_zeros(())
            if self.training and balance_loss is not None:
                balance_term = self.moe_load_balance_weight * balance_loss / self.num_moe_layers
                loss = loss + balance_term
            return (loss, token_loss, balance_term) if self.training else loss
        return logits
