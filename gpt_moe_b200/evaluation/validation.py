"""Validation loss: mean over `val_steps` batches under the "validation" precision phase,
averaged over ranks (summed over pipeline stages) — reference `evaluation/validation.py:9-33`."""
from __future__ import annotations

import torch

from ..parallel import dist_utils as du
from ..runtime.precision import linear_precision_phase


def evaluate_validation(run, val_data_loader, val_steps: int, gpu_batch_size_val: int, seq_len_val: int) -> torch.Tensor:
    run.gpt_model.eval()
    if run.parallel_mode != "pp" or run.master_process:
        val_data_loader.reset()
    trainer = run.trainer
    with linear_precision_phase(run.raw_gpt_model, "validation"), torch.no_grad(), run.ctx:
        val_loss = torch.zeros((), device=run.device)
        for _ in range(val_steps):
            if run.parallel_mode == "pp":
                x, y, docs = run.pipeline_next_batch(val_data_loader, gpu_batch_size_val, seq_len_val)
                step_loss = run.pipeline_non_training_forward(run.gpt_model, x, y, document_ids=docs)
            else:
                x, y, docs = val_data_loader.next_batch()
                x, y, docs = trainer._to_device(x), trainer._to_device(y), trainer._to_device(docs)
                step_loss = run.gpt_model(x, y, document_ids=docs)
            val_loss += step_loss.float() / val_steps
        du.all_reduce(val_loss, op=None if run.parallel_mode == "pp" else "avg")
    return val_loss
