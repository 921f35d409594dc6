"""Kernel warm-up before the timed loop.

The reference runs real train steps on random tokens for every scheduled batch size plus one
validation forward so that compilation and autotuning happen before step 0, then restores model,
optimizer and RNG state (`runtime/warmup.py:12-269`).  Nothing is compiled or autotuned here, but
first launches still pay for CUDA module loading, allocator growth and (on the fused path)
symmetric-memory rendezvous, so the same procedure is kept: warm up, then restore exactly.
"""
from __future__ import annotations

import copy
import time

import torch

from ..parallel import dist_utils as du


def _pipeline_warmup_steps(run, trainer, cfg, num_train_steps: int) -> None:
    """The pipeline form of the warm-up (reference `runtime/warmup.py:12-131`): both stages run real 1F1B optimizer steps
    on random tokens for every scheduled batch size, then the forward-only path across the stages once.  Rank 0 draws the
    tokens; the targets reach stage 1 by the same broadcast as in training."""
    import torch.distributed as dist
    runtime, vocab = trainer.pipeline_runtime, trainer.gpt_config.vocab_size
    uses_docs = run.raw_gpt_model.use_doc_masking

    def random_batch(batch_size: int, seq_len: int):
        if run.master_process:
            ids = torch.randint(0, vocab, (batch_size, seq_len + 1))
            x, y = trainer._to_device(ids[:, :-1].contiguous()), trainer._to_device(ids[:, 1:].contiguous())
        else:
            x, y = None, torch.empty((batch_size, seq_len), dtype=torch.long, device=trainer.device)
        dist.broadcast(y, src=0)
        docs = torch.zeros((batch_size, seq_len), dtype=torch.int32, device=trainer.device) if uses_docs else None
        return x, y, docs

    for batch_size in sorted(set(cfg.batch_size_schedule_values)):
        for _ in range(num_train_steps):
            trainer.engine.zero_grad()
            batches = [random_batch(batch_size, cfg.seq_len_train) for _ in range(cfg.grad_accum_mini_steps)]
            with run.ctx:
                runtime.train_step(batches)
            trainer.engine.step()
    run.gpt_model.eval()
    x, y, docs = random_batch(cfg.gpu_batch_size_val, cfg.seq_len_val)
    with torch.no_grad(), run.ctx:
        runtime.non_training_forward(run.gpt_model, x, y, document_ids=docs)


def kernel_warmup(run, num_train_steps: int = 2) -> float:
    trainer = run.trainer
    if num_train_steps <= 0:
        return 0.0
    cfg = run.training_config
    t0 = time.time()
    model_state = copy.deepcopy(run.raw_gpt_model.state_dict())
    opt_state = {k: copy.deepcopy(o.state_dict()) for k, o in run.optimizers.items()}
    engine_state = trainer.engine.snapshot() if hasattr(trainer.engine, "snapshot") else None
    cpu_rng = torch.get_rng_state()
    cuda_rng = torch.cuda.get_rng_state() if trainer.device_type == "cuda" else None
    saved = (trainer.train_tokens_processed, trainer.schedule_state())
    vocab = trainer.gpt_config.vocab_size
    if run.parallel_mode == "pp":
        _pipeline_warmup_steps(run, trainer, cfg, num_train_steps)
    else:
        for batch_size in sorted(set(cfg.batch_size_schedule_values)):
            trainer.current_batch_size = batch_size
            for _ in range(num_train_steps):
                batches = []
                for _ in range(cfg.grad_accum_mini_steps):
                    ids = torch.randint(0, vocab, (batch_size, cfg.seq_len_train + 1))
                    batches.append((ids[:, :-1].contiguous(), ids[:, 1:].contiguous(), None))
                trainer.train_step(batches, read_losses=False)
        run.gpt_model.eval()
        with torch.no_grad(), run.ctx:
            ids = torch.randint(0, vocab, (cfg.gpu_batch_size_val, cfg.seq_len_val + 1))
            run.gpt_model(trainer._to_device(ids[:, :-1].contiguous()), trainer._to_device(ids[:, 1:].contiguous()))
    # restore
    run.raw_gpt_model.load_state_dict(model_state)
    for k, o in run.optimizers.items():
        o.load_state_dict(opt_state[k])
    if engine_state is not None:
        trainer.engine.restore(engine_state)
    elif hasattr(trainer.engine, "refresh_from_parameters"):
        trainer.engine.refresh_from_parameters()
    torch.set_rng_state(cpu_rng)
    if cuda_rng is not None:
        torch.cuda.set_rng_state(cuda_rng)
    trainer.train_tokens_processed = saved[0]
    for key, value in saved[1].items():
        setattr(trainer, key, value)
    run.raw_gpt_model.set_sliding_window(trainer.current_window_size)
    du.barrier()
    elapsed = du.max_over_ranks(time.time() - t0, run.device)
    if run.master_process:
        message = f"kernel warmup: {elapsed:.2f} s (max over ranks)"
        print(message)
        run.log_buffer.append(message)
    return elapsed
