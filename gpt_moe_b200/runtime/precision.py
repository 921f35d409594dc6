"""Precision policies: parameter dtype casting, autocast context, per-phase linear precision.

Counterpart of the reference's `runtime/precision.py:13-91`.  On the GPU this framework's ops
choose their own compute dtype (bf16 activations, fp32 statistics and accumulators), so the
autocast context matters only for plain torch ops and the CPU path.
"""
from __future__ import annotations

import contextlib
from typing import Any, Dict, Iterator

import torch
import torch.nn as nn

from ..optim.adamw import configure_adamw_moments  # re-exported: same name as the reference's helper

__all__ = ["convert_to_bf16", "configure_adamw_moments", "precision_context", "linear_precision_phase"]


def convert_to_bf16(gpt_model: nn.Module, bf16_weights_params_and_scales: Dict[str, Any],
                    keep_1d_weights_params_and_scales_in_fp32: bool) -> None:
    """Cast all parameters ({"all": object}), or those of the listed module classes / nn.Parameter,
    to bf16; optionally restore 1-D parameters to fp32."""
    if bf16_weights_params_and_scales.get("all") is object:
        selected = list(gpt_model.parameters())
    else:
        classes = tuple(c for c in bf16_weights_params_and_scales.values() if isinstance(c, type))
        module_classes = tuple(c for c in classes if issubclass(c, nn.Module))
        selected = [p for m in gpt_model.modules() if module_classes and isinstance(m, module_classes)
                    for p in m.parameters(recurse=False)]
        if any(c is nn.Parameter for c in classes):
            selected = list(gpt_model.parameters())
    for p in selected:
        if p.is_floating_point() and p.dtype != torch.bfloat16:
            p.data = p.data.to(torch.bfloat16)
    if keep_1d_weights_params_and_scales_in_fp32:
        for p in gpt_model.parameters():
            if p.dim() == 1 and p.dtype == torch.bfloat16:
                p.data = p.data.float()


def precision_context(training_config, device_type: str):
    if training_config.use_all_bf16_and_null_ctx or not training_config.use_bf16_autocast or device_type == "cpu":
        return contextlib.nullcontext()
    return torch.autocast(device_type=device_type, dtype=torch.bfloat16)


@contextlib.contextmanager
def linear_precision_phase(gpt_model, phase: str) -> Iterator[None]:
    previous = gpt_model.precision_phase
    gpt_model.set_precision_phase(phase)
    try:
        yield
    finally:
        gpt_model.set_precision_phase(previous)
