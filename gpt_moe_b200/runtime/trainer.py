"""The training program as a library object.

`Trainer` holds everything the reference's module-level `train.py` script keeps in globals
(`train.py:37-336`): process group, configs, model, engine, optimizers, loaders, schedule state,
timers and the `run` namespace handed to evaluation / sampling / checkpoint helpers.
`Trainer.train_step()` is one optimizer step (`train.py:370-518`): micro-steps with host-to-device
copies from pinned memory, forward/backward, gradient reduction, token-scheduled LR / window /
batch size, optimizer step, and a device-to-host read of the logged losses.
`Trainer.fit()` is the full loop with logging, sampling, evaluations, validation gating,
checkpointing and export (`train.py:370-758`).
"""
from __future__ import annotations

import math
import os
import sys
import time
from types import SimpleNamespace
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..checkpointing import checkpoint as ckpt
from ..config.training import build_resume_config
from ..data.loader import DataLoader, SyntheticLoader
from ..models.attention import qk_scale_debug_string
from ..models.gpt import GPT
from ..optim.adamw import configure_adamw_moments
from ..parallel import dist_utils as du
from ..parallel.ddp_engine import HostEngine
from ..schedules.token import get_next_update_tokens
from . import reporting
from .precision import convert_to_bf16, precision_context
from .watchdog import StepWatchdog


class Trainer:
    def __init__(self, gpt_config, training_config, device_type: Optional[str] = None, quiet: bool = False) -> None:
        self.gpt_config, self.cfg = gpt_config, training_config
        self.device_type = device_type or ("cuda" if torch.cuda.is_available() else "cpu")
        self.rank, self.local_rank, self.world_size = du.env_rank_info()
        du.init_distributed(self.device_type)
        self.device = f"cuda:{self.local_rank}" if self.device_type == "cuda" else "cpu"
        self.master_process = self.rank == 0
        self.quiet = quiet
        cfg = training_config
        self.parallel_mode = cfg.parallel_mode.lower()
        assert self.parallel_mode in ("ddp", "pp"), "parallel_mode must be 'ddp' or 'pp'"
        if self.parallel_mode == "pp":
            assert self.world_size == 2, "pipeline parallelism runs on exactly two ranks"
        assert cfg.checkpoint_interval == -1 or cfg.checkpoint_interval > 0
        assert cfg.checkpoint_best_improvement_interval == -1 or cfg.checkpoint_best_improvement_interval > 0
        assert cfg.full_model_export_interval == -1 or cfg.full_model_export_interval > 0
        assert cfg.max_checkpoints_to_keep > 0
        self.effective_world_size = self.world_size if self.parallel_mode == "ddp" else 1
        cfg.resolve(self.effective_world_size)
        if self.parallel_mode == "pp":
            assert cfg.grad_accum_mini_steps >= self.world_size, "the pipeline schedule needs at least two micro-batches"
        self.ep_size = cfg.expert_parallel_size if (self.parallel_mode == "ddp" and gpt_config.use_moe) else 1
        assert self.world_size % self.ep_size == 0, "expert_parallel_size must divide the world size"

        self.log_buffer: List[str] = []
        if self.master_process:
            self.log_buffer += [f"python: {sys.version}", f"torch: {torch.__version__}", f"torch.cuda: {torch.version.cuda}"]
            reporting.log_source_code(self.log_buffer, include_sources=not quiet)
            self._log(f"per-gpu gradient accumulation mini-steps: {cfg.grad_accum_mini_steps}")
            self._log(f"max train steps: {cfg.max_train_steps:,}")
        torch.set_float32_matmul_precision(cfg.float32_matmul_precision)

        # counters (overwritten on resume)
        self.allow_val = False
        self.start_step = 0
        self.train_tokens_processed = 0
        self.total_train_t = self.total_val_t = self.total_sample_t = self.total_hellaswag_t = self.total_t = 0.0
        self.best_val_loss = float("inf")
        self.best_improvement_count = 0
        epoch = shard_idx = shard_counter = 0
        schedule_state = None
        optimizer_state_dicts = None
        self._resume_rng = None

        seed = cfg.base_seed + (self.rank if self.parallel_mode == "ddp" else 0)
        torch.manual_seed(seed)
        if self.device_type == "cuda":
            torch.cuda.manual_seed(seed)
        self.resume_config = build_resume_config(gpt_config, cfg)

        stage_index = self.rank if self.parallel_mode == "pp" else None
        ep_rank = self.rank % self.ep_size

        def factory() -> GPT:
            # identical initial weights on every rank: construct under the base seed, then restore the rank's stream
            state = torch.get_rng_state()
            torch.manual_seed(cfg.base_seed)
            model = GPT(gpt_config, cfg, stage_index=stage_index, ep_rank=ep_rank, ep_size=self.ep_size)
            torch.set_rng_state(state)
            return model

        if cfg.resume_from_checkpoint:
            loaded = ckpt.load_checkpoint(cfg, gpt_config, self.rank, self.world_size, self.resume_config, model_factory=factory)
            self.start_step = loaded["start_step"]
            self._resume_rng = loaded["rng_state"]
            self.train_tokens_processed = loaded["train_tokens_processed"]
            self.total_train_t, self.total_val_t = loaded["total_train_t"], loaded["total_val_t"]
            self.total_sample_t, self.total_hellaswag_t = loaded["total_sample_t"], loaded["total_hellaswag_t"]
            self.total_t, self.best_val_loss = loaded["total_t"], loaded["best_val_loss"]
            epoch, shard_idx = loaded["epoch"], loaded["current_shard_idx"]
            shard_counter = loaded["grad_accum_mini_steps_per_shard_counter"]
            schedule_state = loaded["schedule_state"]
            self.best_improvement_count, self.allow_val = loaded["best_improvement_count"], loaded["allow_val"]
            optimizer_state_dicts = loaded["optimizer_state_dicts"]
            self.raw_gpt_model = loaded["gpt_model"]
            self._log(f"loaded checkpoint from step {self.start_step - 1}")
            du.barrier()
        else:
            self.raw_gpt_model = factory()
        if getattr(self.raw_gpt_model, "te_roles_on_mxfp8", None):
            self._log("linear backend 'te' (Transformer Engine block scaling) is served by the MXFP8 kernels (e4m3, 32-element E8M0 "
                      "blocks) for: " + ", ".join(self.raw_gpt_model.te_roles_on_mxfp8))
        self.raw_gpt_model.to(self.device)
        if cfg.use_all_bf16_and_null_ctx or cfg.use_bf16_weights_params_or_scales:
            convert_to_bf16(self.raw_gpt_model, cfg.bf16_weights_params_and_scales, cfg.keep_1d_weights_params_and_scales_in_fp32)
        self.gpt_model = self.raw_gpt_model

        # expert-parallel groups: consecutive ranks form one group; ranks at the same position of their groups hold the
        # same experts and form an expert replica group (their expert gradients are summed, nobody else's)
        self.ep_group = self.expert_replica_group = None
        if self.ep_size > 1:
            from ..parallel.ep import attach_expert_parallel
            for start in range(0, self.world_size, self.ep_size):
                ranks = list(range(start, start + self.ep_size))
                group = dist.new_group(ranks)
                if self.rank in ranks:
                    self.ep_group = group
            if self.world_size > self.ep_size:
                for position in range(self.ep_size):
                    ranks = list(range(position, self.world_size, self.ep_size))
                    group = dist.new_group(ranks)
                    if self.rank in ranks:
                        self.expert_replica_group = group
            attach_expert_parallel(self.raw_gpt_model, self.ep_group,
                                   fused=self.device_type == "cuda" and cfg.use_fused_collectives,
                                   capacity_factor=cfg.ep_capacity_factor)

        self.optimizers = self.raw_gpt_model.configure_optimizers(
            cfg.adamw_max_lr, cfg.adamw_betas, cfg.adamw_eps, cfg.adamw_weight_decay, self.device_type,
            master_process=self.master_process and not quiet, log_buffer=self.log_buffer)
        if optimizer_state_dicts is not None:
            if set(self.optimizers) != set(optimizer_state_dicts):
                raise ValueError("checkpoint optimizer names differ from the current run")
            for name, opt in self.optimizers.items():
                # saved files hold the unsharded layout: pick this rank's entries by parameter name
                opt.load_state_dict(ckpt.localize_optimizer_state(self.raw_gpt_model, opt, optimizer_state_dicts[name]))
            du.barrier()
        configure_adamw_moments(self.optimizers["adamw"], cfg.use_bf16_adamw_moments)

        self.engine = self._build_engine()
        self.pipeline_runtime = None
        if self.parallel_mode == "pp":
            from .pipeline import PipelineRuntime
            self.pipeline_runtime = PipelineRuntime(self.raw_gpt_model, self.rank, self.world_size, self.device,
                                                    cfg.grad_accum_mini_steps, self.raw_gpt_model.use_doc_masking)
        self.ctx = precision_context(cfg, self.device_type)

        loader_world = self.world_size if self.parallel_mode == "ddp" else 1
        loader_rank = self.rank if self.parallel_mode == "ddp" else 0
        use_loader = self.parallel_mode == "ddp" or self.master_process
        self.train_data_loader = self.val_data_loader = None
        if use_loader:
            if cfg.use_synthetic_data:
                self.train_data_loader = SyntheticLoader(cfg.gpu_batch_size_train, cfg.seq_len_train, loader_world, loader_rank,
                                                         gpt_config.vocab_size, seed=0, split="train",
                                                         return_document_ids=self.raw_gpt_model.use_doc_masking)
                self.val_data_loader = SyntheticLoader(cfg.gpu_batch_size_val, cfg.seq_len_val, loader_world, loader_rank,
                                                       gpt_config.vocab_size, seed=0, split="val",
                                                       return_document_ids=self.raw_gpt_model.use_doc_masking)
            else:
                common = dict(pad_token_id=gpt_config.pad_token_id, eos_token_id=gpt_config.eos_token_id,
                              return_document_ids=self.raw_gpt_model.use_doc_masking,
                              master_process=self.master_process, log_buffer=self.log_buffer)
                self.train_data_loader = DataLoader(cfg.gpu_batch_size_train, cfg.seq_len_train, loader_world, loader_rank,
                                                    cfg.data_path, "train", epoch=epoch, current_shard_idx=shard_idx,
                                                    grad_accum_mini_steps_per_shard_counter=shard_counter, **common)
                self.val_data_loader = DataLoader(cfg.gpu_batch_size_val, cfg.seq_len_val, loader_world, loader_rank,
                                                  cfg.data_path, "val", shuffle_val_tokens=cfg.shuffle_val_tokens, **common)

        self.run = SimpleNamespace(
            parallel_mode=self.parallel_mode, rank=self.rank, world_size=self.world_size,
            master_process=self.master_process, device=self.device, training_config=cfg,
            gpt_model=self.gpt_model, raw_gpt_model=self.raw_gpt_model, optimizers=self.optimizers,
            tokenizer=None, ctx=self.ctx, log_buffer=self.log_buffer, forward=self.forward_for_evaluation,
            pipeline_next_batch=getattr(self.pipeline_runtime, "next_batch", None),
            pipeline_train_step=getattr(self.pipeline_runtime, "train_step", None),
            pipeline_non_training_forward=getattr(self.pipeline_runtime, "non_training_forward", None),
            trainer=self)
        self._init_schedules(schedule_state)
        self.watchdog = StepWatchdog(cfg.step_deadline_s) if cfg.step_deadline_s > 0 else None
        self._loss_host = None

    # ------------------------------------------------------------------------------------------------
    def _log(self, message: str) -> None:
        if self.master_process:
            if not self.quiet:
                print(message)
            self.log_buffer.append(message)

    def _build_engine(self):
        cfg = self.cfg
        if self.parallel_mode != "ddp":
            return _LocalEngine(self.optimizers)
        if self.device_type == "cuda":
            from ..parallel.fused_engine import build_cuda_engine
            engine = build_cuda_engine(self.raw_gpt_model, cfg, self.optimizers, ep_size=self.ep_size, ep_group=self.ep_group,
                                       expert_replica_group=self.expert_replica_group)
        else:
            engine = HostEngine(self.raw_gpt_model, cfg, self.optimizers, dp_group=None, ep_size=self.ep_size,
                                expert_replica_group=self.expert_replica_group)
        if cfg.resume_from_checkpoint and hasattr(engine, "drop_foreign_state"):
            engine.drop_foreign_state()
        return engine

    def _init_schedules(self, state: Optional[dict]) -> None:
        cfg = self.cfg
        self.swa_schedule_idx = 0
        self.current_window_size = cfg.swa_schedule_values[0]
        self.next_swa_update_tokens = get_next_update_tokens(cfg.swa_schedule_keys, 0, cfg.max_tokens)
        self.batch_schedule_idx = 0
        self.current_batch_size = cfg.batch_size_schedule_values[0]
        self.next_batch_update_tokens = get_next_update_tokens(cfg.batch_size_schedule_keys, 0, cfg.max_tokens)
        self.lr_schedule_idx = 0
        self.next_lr_update_tokens = cfg.lr_schedule[0]["end"]
        if state is not None:
            for key, value in state.items():
                setattr(self, key, value)
        self.raw_gpt_model.set_sliding_window(self.current_window_size)

    def schedule_state(self) -> Dict[str, int]:
        keys = ("swa_schedule_idx", "current_window_size", "next_swa_update_tokens", "batch_schedule_idx",
                "current_batch_size", "next_batch_update_tokens", "lr_schedule_idx", "next_lr_update_tokens")
        return {k: getattr(self, k) for k in keys}

    def forward_for_evaluation(self, model, indices, targets=None, attn_mask=None, ignore_doc_mask=False, document_ids=None):
        if self.parallel_mode == "pp":
            return self.pipeline_runtime.non_training_forward(model, indices, targets, attn_mask, ignore_doc_mask, document_ids)
        return model(indices, targets, attn_mask=attn_mask, ignore_doc_mask=ignore_doc_mask, document_ids=document_ids)

    def _to_device(self, t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if t is None or self.device_type != "cuda" or t.is_cuda:
            return t
        if not t.is_pinned():
            t = t.pin_memory()
        return t.to(self.device, non_blocking=True)

    # ------------------------------------------------------------------------------------------------
    def _nvtx(self, name: str):
        """NVTX range for profilers (`training.nvtx_ranges=True`); a no-op context otherwise."""
        import contextlib
        if self.device_type == "cuda" and getattr(self.cfg, "nvtx_ranges", False):
            return torch.cuda.nvtx.range(name)
        return contextlib.nullcontext()

    def train_step(self, batches: Optional[List[Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]]] = None,
                   read_losses: bool = True) -> Dict[str, float]:
        """One optimizer step.  `batches` (CPU tensors, one per micro-step) overrides the loader."""
        cfg, model, raw = self.cfg, self.gpt_model, self.raw_gpt_model
        accum = cfg.grad_accum_mini_steps
        if self.watchdog is not None:
            self.watchdog.arm()
        if not model.training:                # walking ~1300 modules every step costs milliseconds of host time
            model.train()
        raw.set_precision_phase("training")
        self.engine.zero_grad()
        if accum > 1:
            raw.prepare_fp8_weights()

        if self.train_tokens_processed >= self.next_batch_update_tokens and self.batch_schedule_idx + 1 < len(cfg.batch_size_schedule_keys):
            self.batch_schedule_idx += 1
            self.current_batch_size = cfg.batch_size_schedule_values[self.batch_schedule_idx]
            self.next_batch_update_tokens = get_next_update_tokens(cfg.batch_size_schedule_keys, self.batch_schedule_idx, cfg.max_tokens)
        bs = self.current_batch_size

        # token-based learning rate: it depends only on the tokens processed before this step, so it is set before the backward
        # pass (the fused engine starts optimizer work for a block as soon as that block's gradients exist)
        if self.train_tokens_processed >= self.next_lr_update_tokens and self.lr_schedule_idx + 1 < len(cfg.lr_schedule):
            self.lr_schedule_idx += 1
            self.next_lr_update_tokens = cfg.lr_schedule[self.lr_schedule_idx]["end"]
        spec = cfg.lr_schedule[self.lr_schedule_idx]
        adamw_lr = spec["fn"](self.train_tokens_processed - spec["start"], **spec["kwargs"])
        for group in self.optimizers["adamw"].param_groups:
            group["lr"] = adamw_lr
        if "muon" in self.optimizers:
            for group in self.optimizers["muon"].param_groups:
                group["lr"] = adamw_lr * raw.muon_lr_scale

        if self.parallel_mode == "pp":
            pipeline_batches = [self.pipeline_runtime.next_batch(self.train_data_loader, bs, cfg.seq_len_train) for _ in range(accum)]
            with self.ctx:
                train_losses = self.pipeline_runtime.train_step(pipeline_batches)
            du.all_reduce(train_losses)
        else:
            train_losses = torch.zeros(3, device=self.device)
            for mini_step in range(accum):
                x, y, docs = batches[mini_step] if batches is not None else self.train_data_loader.next_batch()
                x, y = self._to_device(x[:bs]), self._to_device(y[:bs])
                docs = self._to_device(docs[:bs]) if docs is not None else None
                last = mini_step == accum - 1
                with self.ctx, self._nvtx(f"forward_backward[{mini_step}]"):
                    loss, token_loss, balance = self.engine.forward_backward(model, x, y, docs, 1.0 / accum, last)
                train_losses += torch.stack((loss.detach().float(), token_loss.detach().float(), balance.detach().float())) / accum
            du.all_reduce(train_losses, op="avg")

        # token-based window schedule
        if self.train_tokens_processed >= self.next_swa_update_tokens and self.swa_schedule_idx + 1 < len(cfg.swa_schedule_keys):
            self.swa_schedule_idx += 1
            self.current_window_size = cfg.swa_schedule_values[self.swa_schedule_idx]
            self.next_swa_update_tokens = get_next_update_tokens(cfg.swa_schedule_keys, self.swa_schedule_idx, cfg.max_tokens)
        raw.set_sliding_window(self.current_window_size)
        raw.clear_fp8_weights()
        loss_ready = None
        if read_losses and self.device_type == "cuda":
            # the losses are final once the backward pass is issued: their copy to pinned host memory is queued BEFORE the
            # optimizer kernels, so the host gets the numbers (and starts issuing the next step) while the optimizer still runs
            if self._loss_host is None:
                self._loss_host = torch.empty(3, dtype=torch.float32, pin_memory=True)
            self._loss_host.copy_(train_losses, non_blocking=True)
            loss_ready = torch.cuda.Event()
            loss_ready.record()
        with self._nvtx("optimizer_step"):
            self.engine.step()

        out = {"adamw_lr": adamw_lr, "tokens": bs * cfg.seq_len_train * self.effective_world_size * accum}
        if read_losses:
            if loss_ready is not None:
                loss_ready.synchronize()
                vals = self._loss_host.tolist()
            else:
                vals = train_losses.tolist()
            out.update(loss=vals[0], token_loss=vals[1], balance_term=vals[2])
        self.train_tokens_processed += out["tokens"]
        if self.watchdog is not None:
            self.watchdog.disarm()
        return out

    # ------------------------------------------------------------------------------------------------
    def save(self, step: int, train_loss: float, val_loss: Optional[float]) -> Optional[str]:
        cfg = self.cfg
        position = [(self.train_data_loader.epoch, self.train_data_loader.current_shard_idx,
                     self.train_data_loader.grad_accum_mini_steps_per_shard_counter) if self.master_process else None]
        if du.is_dist() and self.world_size > 1:
            dist.broadcast_object_list(position, src=0)
        rng = {"cpu": torch.get_rng_state(), "cuda": torch.cuda.get_rng_state() if self.device_type == "cuda" else torch.empty(0, dtype=torch.uint8)}
        if self.parallel_mode == "ddp" and self.world_size > 1:
            rngs = [None] * self.world_size if self.master_process else None
            dist.gather_object(rng, rngs, dst=0)
        else:
            rngs = [rng]
        if hasattr(self.engine, "full_model_state"):      # engines with sharded fp32 masters gather them
            model_state = self.engine.full_model_state()
        else:
            model_state = ckpt.gather_full_state_dict(self.raw_gpt_model, self.ep_group)
        opt_states = self.engine.full_optimizer_state_dicts() if hasattr(self.engine, "full_optimizer_state_dicts") else None
        path = None
        if self.parallel_mode == "pp" or self.master_process:
            path = ckpt.save_checkpoint(
                cfg.checkpoint_dir, self.raw_gpt_model, self.log_buffer, step=step, rng_states_by_rank=rngs,
                train_loss=train_loss, val_loss=val_loss, train_tokens_processed=self.train_tokens_processed,
                total_train_t=self.total_train_t, total_val_t=self.total_val_t, total_sample_t=self.total_sample_t,
                total_hellaswag_t=self.total_hellaswag_t, total_t=self.total_t, best_val_loss=float(self.best_val_loss),
                epoch=position[0][0], current_shard_idx=position[0][1], grad_accum_mini_steps_per_shard_counter=position[0][2],
                optimizers=self.optimizers, parallel_mode=self.parallel_mode, world_size=self.world_size, rank=self.rank,
                resume_config=self.resume_config, schedule_state=self.schedule_state(),
                best_improvement_count=self.best_improvement_count, allow_val=self.allow_val,
                model_state=model_state, optimizer_state_dicts=opt_states)
        du.barrier()
        if self.master_process:
            ckpt.keep_latest_checkpoints(cfg.checkpoint_dir, cfg.max_checkpoints_to_keep, self.log_buffer)
        du.barrier()
        return path

    def _sync(self) -> None:
        if self.device_type == "cuda":
            torch.cuda.synchronize()

    def fit(self, max_steps: Optional[int] = None) -> None:
        """The full training loop (reference `train.py:337-758`)."""
        from ..evaluation.validation import evaluate_validation
        cfg, raw = self.cfg, self.raw_gpt_model
        run = self.run
        run.tokenizer = cfg.get_tokenizer() if (cfg.run_sampling or cfg.run_benchmarks or cfg.run_gsm8k) else None
        if cfg.run_benchmarks:
            from ..evaluation.hellaswag import load_hellaswag_data
            load_hellaswag_data(run)
        if cfg.run_gsm8k:
            from ..evaluation.gsm8k import load_gsm8k_data
            load_gsm8k_data(run)
        if self.master_process:
            reporting.save_config_info(run, cfg, self.gpt_config)
        reporting.log_parameter_counts(run, self.gpt_config)
        reporting.flush_log(run)
        from .warmup import kernel_warmup
        kernel_warmup(run, num_train_steps=cfg.kernel_warmup_train_steps)
        if self._resume_rng is not None:
            torch.set_rng_state(self._resume_rng["cpu"])
            if self.device_type == "cuda" and self._resume_rng["cuda"].numel():
                torch.cuda.set_rng_state(self._resume_rng["cuda"])
        last_step = cfg.max_train_steps if max_steps is None else min(cfg.max_train_steps, self.start_step + max_steps)
        try:
            for step in range(self.start_step, last_step):
                final = step == last_step - 1
                self._sync()
                t0 = time.time()
                stats = self.train_step()
                self._sync()
                dt = du.max_over_ranks(time.time() - t0, self.device) if self.parallel_mode == "pp" else time.time() - t0
                self.total_train_t += dt
                self.total_t += dt
                tl = stats["loss"]
                qk = ""
                if raw.use_qk_norm and raw.use_qk_debug_log:
                    if self.parallel_mode == "pp":
                        parts = [None] * self.world_size
                        dist.all_gather_object(parts, qk_scale_debug_string(raw))
                        qk = "".join(f"stage {r}: {v}" for r, v in enumerate(parts))
                    elif self.master_process:
                        qk = qk_scale_debug_string(raw)
                self._log(
                    f"step: {step:,} | train loss: {tl:.8f} | train token loss: {stats['token_loss']:.8f} | "
                    f"train balance term: {stats['balance_term']:.8f} | train ppl: {math.exp(min(stats['token_loss'], 700)):,.2f} | "
                    f"train step time: {1000 * dt:,.2f} ms | adamw lr: {stats['adamw_lr']:.8f} | "
                    f"tok/s: {stats['tokens'] / dt:,.2f} | total toks: {self.train_tokens_processed:,} | "
                    f"total train time: {self.total_train_t / 60:,.2f} min | sw size: {self.current_window_size} | "
                    f"{qk}batch size: {self.current_batch_size:,}")

                if cfg.run_sampling and ((step % cfg.sample_interval == 0 and step > 0) or final):
                    from ..sampling.sample import get_sample_token_count, sample
                    self._sync(); t = time.time()
                    sample(run, cfg.sample_sequences, max_new_tokens=get_sample_token_count(step))
                    self._sync(); d = time.time() - t
                    self.total_sample_t += d; self.total_t += d
                    self._log(f"step: {step:,} | sampling time: {d:,.2f} s")
                if cfg.run_benchmarks and ((step % cfg.hellaswag_interval == 0 and step > 0) or final):
                    from ..evaluation.hellaswag import evaluate_hellaswag_standard
                    self._sync(); t = time.time()
                    acc = evaluate_hellaswag_standard(run)
                    self._sync(); d = time.time() - t
                    self.total_hellaswag_t += d; self.total_t += d
                    self._log(f"step: {step:,} | HellaSwag acc: {acc:.4f} | HellaSwag time: {d:,.2f} s")

                if tl + cfg.train_val_margin <= cfg.val_target and not self.allow_val:
                    self.allow_val = True
                    self._log(f"val enabled at step {step} - {tl} train loss")
                checkpoint_val_loss, improved, stop = None, False, False
                if (self.allow_val and step % cfg.val_interval == 0 and step > 0) or final:
                    self._sync(); t = time.time()
                    self._log(f"resetting val loader at step {step}")
                    val_loss = float(evaluate_validation(run, self.val_data_loader, cfg.val_steps, cfg.gpu_batch_size_val, cfg.seq_len_val))
                    checkpoint_val_loss = val_loss
                    if val_loss < self.best_val_loss:
                        self.best_val_loss, improved = val_loss, True
                        self.best_improvement_count += 1
                        self._log(f"new best val loss: {val_loss:.8f}")
                        reporting.flush_log(run)
                        du.barrier()
                    self._sync(); d = time.time() - t
                    self.total_val_t += d; self.total_t += d
                    self._log(f"step: {step:,} | val loss: {val_loss:.8f} | val ppl: {math.exp(min(val_loss, 700)):,.2f} | val time: {1000 * d:,.2f} ms")
                    if val_loss <= cfg.val_target:
                        self._log(f"val loss {val_loss:.8f} reached target {cfg.val_target}")
                        stop = True

                periodic = cfg.checkpoint_interval > 0 and (step + 1) % cfg.checkpoint_interval == 0
                best = improved and cfg.checkpoint_best_improvement_interval > 0 and \
                    self.best_improvement_count % cfg.checkpoint_best_improvement_interval == 0
                weights_path = None
                if cfg.enable_checkpointing and (periodic or best):
                    weights_path = self.save(step, tl, checkpoint_val_loss)
                export_due = (cfg.export_full_model_at_end and (stop or final)) or \
                    (cfg.full_model_export_interval > 0 and (step + 1) % cfg.full_model_export_interval == 0)
                if export_due:
                    self._export(step, weights_path)
                if cfg.run_gsm8k and (stop or final or (cfg.gsm8k_interval > 0 and step > 0 and step % cfg.gsm8k_interval == 0)):
                    from ..evaluation.gsm8k import evaluate_gsm8k
                    self._sync(); t = time.time()
                    acc = evaluate_gsm8k(run)
                    self._sync(); d = time.time() - t
                    self.total_t += d
                    self._log(f"step: {step:,} | GSM8K acc: {acc:.4f} | GSM8K time: {d:,.2f} s")
                if stop:
                    break
        except Exception as exc:
            if self.master_process:
                import traceback
                print(f"[rank {self.rank}] unhandled exception: {exc}")
                traceback.print_exc()
            raise
        finally:
            raw.clear_fp8_weights()
            reporting.flush_log(run)

    def _export(self, step: int, weights_path: Optional[str]) -> None:
        cfg = self.cfg
        if self.parallel_mode == "pp":
            stage_path = weights_path or ckpt.save_stage_weights_for_export(self.raw_gpt_model, cfg.model_export_dir, step, self.rank)
            paths = [None] * self.world_size if self.master_process else None
            dist.gather_object(stage_path, paths, dst=0)
            if self.master_process:
                out = ckpt.export_full_model_pp(paths, self.resume_config, cfg.model_export_dir, step, self.current_window_size)
            du.barrier()
            if weights_path is None:
                os.remove(stage_path)
            du.barrier()
        else:
            state = ckpt.gather_full_state_dict(self.raw_gpt_model, self.ep_group) if weights_path is None else None
            if self.master_process:
                out = ckpt.export_full_model_ddp(self.raw_gpt_model, self.resume_config, cfg.model_export_dir, step,
                                                 self.current_window_size, weights_path, model_state=state)
        if self.master_process:
            self._log(f"exported full model to: {out}")

    def close(self) -> None:
        if self.watchdog is not None:
            self.watchdog.stop()
        if self.device_type == "cuda":
            from ..ops import cuda_ops
            cuda_ops.check_status()               # the per-step check is deferred by one step: surface the last one now
        du.barrier()
        if self.ep_size > 1 and self.device_type == "cuda":
            from ..parallel.ep_fused import release_workspaces
            release_workspaces()
        if du.is_dist():
            dist.destroy_process_group()


class _LocalEngine:
    """Optimizer stepping without data parallelism (pipeline stages own disjoint parameters)."""

    def __init__(self, optimizers) -> None:
        self.optimizers = optimizers

    def zero_grad(self) -> None:
        for opt in self.optimizers.values():
            opt.zero_grad(set_to_none=True)

    def step(self) -> None:
        for opt in self.optimizers.values():
            opt.step()
