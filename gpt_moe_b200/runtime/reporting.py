"""Run logging: buffered log file, environment snapshot, config dump, parameter counts.

Counterpart of the reference's `runtime/reporting.py:12-136`: rank 0 keeps an in-memory
`log_buffer` that is appended to `log.txt` at start-up, on every new best validation loss and at
exit; the start-up snapshot records the git commit, `nvidia-smi`, CPU and memory information and
the text of every source file so a log is self-describing.
"""
from __future__ import annotations

import os
import subprocess
from dataclasses import asdict, is_dataclass
from typing import List

import torch

from ..parallel import dist_utils as du


def flush_log(run) -> None:
    if not run.master_process or not run.log_buffer:
        return
    os.makedirs(os.path.dirname(run.training_config.log_filename) or ".", exist_ok=True)
    with open(run.training_config.log_filename, "a") as f:
        f.write("\n".join(run.log_buffer) + "\n")
    run.log_buffer.clear()


def _command(args: List[str]) -> str:
    try:
        return subprocess.run(args, capture_output=True, text=True, timeout=20).stdout.strip()
    except Exception as exc:  # tool not present on this machine
        return f"<{args[0]} unavailable: {exc}>"


def log_source_code(log_buffer: List[str], include_sources: bool = True) -> None:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    commit = _command(["git", "-C", root, "rev-parse", "HEAD"])
    dirty = bool(_command(["git", "-C", root, "status", "--porcelain"]))
    log_buffer.append(f"git commit: {commit}{' (dirty)' if dirty else ''}")
    log_buffer.append(_command(["nvidia-smi"]))
    log_buffer.append(_command(["lscpu"]))
    log_buffer.append(_command(["free", "-b"]))
    for limit in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/cpu.max"):
        if os.path.exists(limit):
            with open(limit) as f:
                log_buffer.append(f"{limit}: {f.read().strip()}")
    if not include_sources:
        return
    for folder, _, files in os.walk(root):
        parts = os.path.relpath(folder, root).split(os.sep)
        # hidden / private folders, run outputs and vendored trees are not part of the program being logged
        if any((part.startswith((".", "_")) and part != ".") or part.endswith("_out") for part in parts) or parts[0] in SKIPPED_TOP_LEVEL:
            continue
        for name in sorted(files):
            if name.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                path = os.path.join(folder, name)
                with open(path, errors="replace") as f:
                    log_buffer.append(f"{'=' * 20} {os.path.relpath(path, root)} {'=' * 20}\n{f.read()}")


SKIPPED_TOP_LEVEL = ("baseline", "configs_and_logs", "checkpoints", "model_exports", "profiles")


def save_config_info(run, training_config, gpt_config) -> None:
    os.makedirs(training_config.config_and_log_dir, exist_ok=True)
    with open(training_config.config_filename, "w") as f:
        for title, cfg in (("GPTConfig", gpt_config), ("TrainingConfig", training_config)):
            f.write(f"[{title}]\n")
            items = asdict(cfg) if is_dataclass(cfg) else vars(cfg)
            for key, value in items.items():
                if key in ("hf_token", "tokenizer"):
                    continue
                f.write(f"{key} = {value!r}\n")
            f.write("\n")


def count_parameters(model, gpt_config) -> tuple:
    """(total parameters, parameters active per token).  Active = total minus the routed experts a
    token does not visit."""
    total = sum(p.numel() for p in model.parameters())
    active = total
    if gpt_config.use_moe:
        expert = sum(p.numel() for n, p in model.named_parameters() if ".mlp.experts." in n)
        local_experts = max(1, sum(1 for n, _ in model.named_parameters() if n.endswith("up_proj.weight") and ".mlp.experts." in n))
        layers = len(model.transformer.h)
        per_expert = expert / local_experts
        active = total - expert + per_expert * gpt_config.moe_top_k * layers
    return int(total), int(active)


def log_parameter_counts(run, gpt_config) -> None:
    total, active = count_parameters(run.raw_gpt_model, gpt_config)
    if run.parallel_mode == "pp" and du.is_dist():
        t = torch.tensor([total, active], dtype=torch.int64, device=run.device)
        du.all_reduce(t)
        total, active = int(t[0]), int(t[1])
    if run.master_process:
        for message in (f"total parameters: {total:,}", f"active parameters per token: {active:,}"):
            print(message)
            run.log_buffer.append(message)
