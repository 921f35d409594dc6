"""Checkpoint save / resume / export in the reference's on-disk layout.

Files (reference `checkpointing/checkpoint.py:34-258`):
  model_step_{step:07d}_{val_%.4f|val_na}_train_%.4f[_stage_{r}].safetensors   model weights
  training_state_step_{step:07d}[_stage_{r}].pt                                 everything else
  full_model_step_{step:07d}.safetensors + _config.json                         export
The weights file holds the plain module's state dict (tied weights stored once); the training
state is a `torch.save`d dict with `format_version == 2` and the key set listed in
`TRAINING_STATE_KEYS`.  Resume demands equality of `resume_config` (only
`use_bf16_adamw_moments` may differ).

Sharded runs write the UNSHARDED layout: with expert parallelism every rank contributes its
experts under their global indices (`gather_full_state_dict`), and Muon momentum buffers are
saved full-shape, so files remain interchangeable with single-GPU runs and with the reference.
"""
from __future__ import annotations

import json
import os
import re
import shutil
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from safetensors.torch import load_file, save_file

TRAINING_STATE_KEYS = (
    "format_version", "parallel_mode", "world_size", "rank", "resume_config", "schedule_state",
    "best_improvement_count", "allow_val", "step", "rng_states_by_rank", "train_tokens_processed",
    "total_train_t", "total_val_t", "total_sample_t", "total_hellaswag_t", "total_t", "best_val_loss",
    "epoch", "current_shard_idx", "grad_accum_mini_steps_per_shard_counter", "optimizer_state_dicts",
)


def unwrap(model: nn.Module) -> nn.Module:
    """Strip engine / DDP / compile wrappers down to the plain GPT module."""
    while True:
        inner = getattr(model, "module", None) or getattr(model, "_orig_mod", None)
        if inner is None:
            return model
        model = inner


def model_state_for_save(model: nn.Module) -> Dict[str, torch.Tensor]:
    """State dict with shared storage stored once (what safetensors' `save_model` writes)."""
    state, seen = {}, {}
    for key, tensor in unwrap(model).state_dict().items():
        ptr = (tensor.data_ptr(), tuple(tensor.shape))
        if ptr in seen and tensor.numel() > 0:
            continue
        seen[ptr] = key
        state[key] = tensor.detach().to("cpu").contiguous()
    return state


def gather_full_state_dict(model: nn.Module, ep_group=None) -> Dict[str, torch.Tensor]:
    """Local state dict, plus (with expert parallelism) every other rank's expert tensors."""
    state = model_state_for_save(model)
    if ep_group is None or dist.get_world_size(ep_group) == 1:
        return state
    local_experts = {k: v for k, v in state.items() if ".mlp.experts." in k}
    gathered: List[Optional[Dict[str, torch.Tensor]]] = [None] * dist.get_world_size(ep_group)
    dist.all_gather_object(gathered, local_experts, group=ep_group)
    for part in gathered:
        state.update(part)
    return state


_EXPERT_RE = re.compile(r"^(.*\.mlp\.experts\.)(\d+)(\..*)$")


def _expert_key(name: str) -> str:
    """Parameter name with the expert index blanked: experts of one layer share it."""
    m = _EXPERT_RE.match(name)
    return name if m is None else f"{m.group(1)}*{m.group(3)}"


def global_param_order(model: nn.Module) -> List[str]:
    """Parameter names of the UNSHARDED model in its `named_parameters()` order.  With expert parallelism the local
    module holds only some experts of every MoE layer; the others are filled in under their global indices, at the
    place the unsharded module lists them (all experts of a layer, in index order, with one expert's parameter order)."""
    model = unwrap(model)
    experts_of_layer: Dict[str, int] = {}
    for mod_name, module in model.named_modules():
        if hasattr(module, "num_experts") and hasattr(module, "experts"):
            experts_of_layer[mod_name + ".experts."] = int(module.num_experts)
    names = [n for n, _ in model.named_parameters()]
    out: List[str] = []
    done = set()
    for i, name in enumerate(names):
        m = _EXPERT_RE.match(name)
        if m is None:
            out.append(name)
            continue
        prefix = m.group(1)
        if prefix in done:
            continue
        done.add(prefix)
        first = m.group(2)
        suffixes = [mm.group(3) for mm in (_EXPERT_RE.match(n) for n in names[i:]) if mm and mm.group(1) == prefix and mm.group(2) == first]
        for e in range(experts_of_layer.get(prefix, 0)):
            out.extend(f"{prefix}{e}{suffix}" for suffix in suffixes)
    return out


def _optimizer_layout(model: nn.Module, optimizer: torch.optim.Optimizer):
    """(local names per param group, global names per param group, {global name: global index}) of one optimizer: the
    global lists are what the optimizer of the unsharded model would hold, in its order."""
    name_of = {id(p): n for n, p in unwrap(model).named_parameters()}
    local_groups = [[name_of[id(p)] for p in g["params"]] for g in optimizer.param_groups]
    order = global_param_order(model)
    global_groups, index = [], {}
    for local in local_groups:
        keys = {_expert_key(n) for n in local}
        names = [n for n in order if _expert_key(n) in keys]
        for n in names:
            index[n] = len(index)
        global_groups.append(names)
    return local_groups, global_groups, index


def merge_optimizer_state(model: nn.Module, optimizer: torch.optim.Optimizer, contributes, group=None) -> Dict[str, Any]:
    """State dict of `optimizer` in the unsharded torch layout, assembled from all ranks of `group`.

    Every rank hands in the state of the parameters for which `contributes(name)` is true on that rank (the owner of a
    sharded matrix; one holder of each expert); entries are matched by parameter NAME, so expert-parallel ranks whose
    local parameter lists differ merge correctly, and are re-keyed by the parameter's position in the unsharded model.
    Collective over `group`."""
    local_groups, global_groups, index = _optimizer_layout(model, optimizer)
    sd = optimizer.state_dict()
    flat_local = [n for names in local_groups for n in names]
    mine = {flat_local[i]: _state_to_cpu(state) for i, state in sd["state"].items() if contributes(flat_local[i])}
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        parts: List[Optional[dict]] = [None] * dist.get_world_size(group)
        dist.all_gather_object(parts, mine, group=group)
        merged: Dict[str, Any] = {}
        for part in parts:
            for name, state in part.items():
                merged.setdefault(name, state)
    else:
        merged = mine
    state = {index[name]: value for name, value in merged.items() if name in index}
    param_groups = []
    for saved, names in zip(sd["param_groups"], global_groups):
        param_groups.append({**saved, "params": [index[n] for n in names]})
    return {"state": dict(sorted(state.items())), "param_groups": param_groups}


def localize_optimizer_state(model: nn.Module, optimizer: torch.optim.Optimizer, state_dict: Dict[str, Any]) -> Dict[str, Any]:
    """Inverse of `merge_optimizer_state` for loading: the entries of an unsharded-layout state dict that belong to this
    rank's parameters, keyed by the local optimizer's indices."""
    local_groups, _, index = _optimizer_layout(model, optimizer)
    state, param_groups, cursor = {}, [], 0
    for saved, names in zip(state_dict["param_groups"], local_groups):
        ids = list(range(cursor, cursor + len(names)))
        cursor += len(names)
        for i, name in zip(ids, names):
            entry = state_dict["state"].get(index[name])
            if entry is not None:
                state[i] = entry
        param_groups.append({**saved, "params": ids})
    return {"state": state, "param_groups": param_groups}


def _state_to_cpu(obj):
    if isinstance(obj, torch.Tensor):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _state_to_cpu(v) for k, v in obj.items()}
    return obj


def keep_latest_checkpoints(checkpoint_dir: str, max_checkpoints_to_keep: int, log_buffer: List[str]) -> None:
    by_step: Dict[int, List[str]] = {}
    for name in os.listdir(checkpoint_dir):
        m = re.fullmatch(r"(?:model|training_state)_step_(\d+).*\.(?:safetensors|pt)", name)
        if m:
            by_step.setdefault(int(m.group(1)), []).append(name)
    for step in sorted(by_step)[:-max_checkpoints_to_keep]:
        for name in by_step[step]:
            path = os.path.join(checkpoint_dir, name)
            os.remove(path)
            message = f"removed checkpoint file: {path}"
            print(message)
            log_buffer.append(message)


def save_checkpoint(checkpoint_dir: str, gpt_model: nn.Module, log_buffer: List[str], step: int,
                    rng_states_by_rank: List[Dict[str, torch.Tensor]], val_loss: Optional[float], train_loss: float,
                    train_tokens_processed: int, total_train_t: float, total_val_t: float, total_sample_t: float,
                    total_hellaswag_t: float, total_t: float, best_val_loss: float, epoch: int, current_shard_idx: int,
                    grad_accum_mini_steps_per_shard_counter: int, optimizers: Dict[str, torch.optim.Optimizer],
                    parallel_mode: str, world_size: int, rank: int, resume_config: Dict[str, Any],
                    schedule_state: Dict[str, Any], best_improvement_count: int, allow_val: bool,
                    model_state: Optional[Dict[str, torch.Tensor]] = None,
                    optimizer_state_dicts: Optional[Dict[str, Any]] = None) -> str:
    os.makedirs(checkpoint_dir, exist_ok=True)
    val_part = f"val_{val_loss:.4f}" if val_loss is not None else "val_na"
    stage = f"_stage_{rank}" if parallel_mode == "pp" else ""
    weights_path = os.path.join(checkpoint_dir, f"model_step_{step:07d}_{val_part}_train_{train_loss:.4f}{stage}.safetensors")
    save_file(model_state if model_state is not None else model_state_for_save(gpt_model), weights_path)
    message = f"saved model weights locally in: {weights_path}"
    print(message)
    log_buffer.append(message)
    if optimizer_state_dicts is None:
        optimizer_state_dicts = {name: opt.state_dict() for name, opt in optimizers.items()}
    training_state = {
        "format_version": 2, "parallel_mode": parallel_mode, "world_size": world_size, "rank": rank,
        "resume_config": resume_config, "schedule_state": schedule_state,
        "best_improvement_count": best_improvement_count, "allow_val": allow_val, "step": step,
        "rng_states_by_rank": rng_states_by_rank, "train_tokens_processed": train_tokens_processed,
        "total_train_t": total_train_t, "total_val_t": total_val_t, "total_sample_t": total_sample_t,
        "total_hellaswag_t": total_hellaswag_t, "total_t": total_t, "best_val_loss": best_val_loss,
        "epoch": epoch, "current_shard_idx": current_shard_idx,
        "grad_accum_mini_steps_per_shard_counter": grad_accum_mini_steps_per_shard_counter,
        "optimizer_state_dicts": optimizer_state_dicts,
    }
    state_path = os.path.join(checkpoint_dir, f"training_state_step_{step:07d}{stage}.pt")
    tmp = state_path + ".tmp"
    torch.save(training_state, tmp)
    os.replace(tmp, state_path)            # a crash mid-write never leaves a truncated state file
    message = f"saved training state locally in: {state_path}"
    print(message)
    log_buffer.append(message)
    return weights_path


def _resolve_file(path: str, training_config) -> str:
    if os.path.isfile(path):
        return path
    from huggingface_hub import hf_hub_download
    return hf_hub_download(repo_id=training_config.hub_repo_id, filename=path, token=training_config.hf_token, repo_type="model")


def load_model_state(gpt_model: nn.Module, state: Dict[str, torch.Tensor]) -> None:
    """Strict load; fills in the missing half of a tied embedding/head pair and drops experts other
    ranks own (reference `checkpoint.py:177-183`)."""
    model = unwrap(gpt_model)
    if getattr(model, "use_tied_embeddings", False):
        e, h = "transformer.wte.weight", "lm_head.weight"
        if e not in state and h in state:
            state[e] = state[h]
        elif h not in state and e in state:
            state[h] = state[e]
    own = set(model.state_dict().keys())
    state = {k: v for k, v in state.items() if k in own or ".mlp.experts." not in k}
    model.load_state_dict(state, strict=True)


def load_checkpoint(training_config, gpt_config, rank: int, world_size: int, resume_config: Dict[str, Any],
                    model_factory=None) -> Dict[str, Any]:
    """Validate and load; returns a dict with `start_step`, `rng_state`, every counter of the
    training state, `optimizer_state_dicts` and the constructed `gpt_model`."""
    mode = training_config.parallel_mode.lower()
    weights_path, state_path = training_config.resume_checkpoint_path, training_config.resume_state_dict_path
    if not weights_path or not state_path:
        raise ValueError("both resume checkpoint paths must be configured")
    if mode == "pp":
        if "{rank}" not in weights_path or "{rank}" not in state_path:
            raise ValueError("pipeline resume paths must contain {rank} for the stage number")
        weights_path, state_path = weights_path.format(rank=rank), state_path.format(rank=rank)
    weights_path, state_path = _resolve_file(weights_path, training_config), _resolve_file(state_path, training_config)

    ts = torch.load(state_path, map_location="cpu", weights_only=False)
    if ts.get("format_version") != 2:
        raise ValueError("checkpoint format version 2 is required")
    if ts["parallel_mode"] != mode:
        raise ValueError("checkpoint parallel mode differs from the current configuration")
    if ts["world_size"] != world_size:
        raise ValueError("checkpoint GPU count differs from the current run")
    if mode == "pp" and ts["rank"] != rank:
        raise ValueError("checkpoint stage number differs from this rank")
    saved = {**ts["resume_config"], "training": {**ts["resume_config"]["training"],
                                                   "use_bf16_adamw_moments": training_config.use_bf16_adamw_moments}}
    if _canonical(saved) != _canonical(resume_config):
        raise ValueError("checkpoint model or training configuration differs from the current run")

    if model_factory is None:
        from ..models.gpt import GPT
        model_factory = lambda: GPT(gpt_config, training_config, stage_index=rank if mode == "pp" else None)
    gpt_model = model_factory()
    load_model_state(gpt_model, load_file(weights_path, device="cpu"))

    rngs = ts["rng_states_by_rank"]
    if len(rngs) != (world_size if mode == "ddp" else 1):
        raise ValueError("checkpoint RNG state count differs from the current run")
    out = {k: ts[k] for k in TRAINING_STATE_KEYS if k in ts}
    out["start_step"] = ts["step"] + 1
    out["rng_state"] = rngs[rank if mode == "ddp" else 0]
    out["gpt_model"] = gpt_model
    return out


def _canonical(obj: Any) -> Any:
    """Tuples and lists compare equal after a save/load round trip."""
    if isinstance(obj, dict):
        return {k: _canonical(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_canonical(v) for v in obj]
    return obj


def _write_export_config(resume_config: Dict[str, Any], export_dir: str, step: int, window: int) -> None:
    with open(os.path.join(export_dir, f"full_model_step_{step:07d}_config.json"), "w") as f:
        json.dump({**resume_config, "sliding_window_size": window}, f, indent=2, default=str)


def save_stage_weights_for_export(gpt_model: nn.Module, export_dir: str, step: int, rank: int) -> str:
    path = os.path.join(export_dir, f"stage_weights_step_{step:07d}_stage_{rank}.safetensors")
    if os.path.exists(path):
        raise FileExistsError(path)
    save_file(model_state_for_save(gpt_model), path)
    return path


def export_full_model_ddp(gpt_model: nn.Module, resume_config: Dict[str, Any], export_dir: str, step: int,
                          current_window_size: int, checkpoint_model_path: Optional[str],
                          model_state: Optional[Dict[str, torch.Tensor]] = None) -> str:
    os.makedirs(export_dir, exist_ok=True)
    path = os.path.join(export_dir, f"full_model_step_{step:07d}.safetensors")
    if os.path.exists(path):
        raise FileExistsError(path)
    if checkpoint_model_path is not None:
        try:
            os.link(checkpoint_model_path, path)
        except OSError:
            shutil.copyfile(checkpoint_model_path, path)
    else:
        save_file(model_state if model_state is not None else model_state_for_save(gpt_model), path)
    _write_export_config(resume_config, export_dir, step, current_window_size)
    return path


def export_full_model_pp(stage_paths: List[str], resume_config: Dict[str, Any], export_dir: str, step: int,
                         current_window_size: int) -> str:
    """Merge the two stage files, renumbering stage 1's blocks by n_layers // 2."""
    if len(stage_paths) != 2:
        raise ValueError("full-model export requires both pipeline stage files")
    path = os.path.join(export_dir, f"full_model_step_{step:07d}.safetensors")
    if os.path.exists(path):
        raise FileExistsError(path)
    split = resume_config["model"]["n_layers"] // 2
    merged: Dict[str, torch.Tensor] = {}
    for stage, stage_path in enumerate(stage_paths):
        for key, value in load_file(stage_path, device="cpu").items():
            if stage == 1 and key.startswith("transformer.h."):
                _, _, idx, tail = key.split(".", 3)
                key = f"transformer.h.{int(idx) + split}.{tail}"
            if key in merged:
                raise ValueError(f"duplicate model weight during pipeline export: {key}")
            merged[key] = value
    save_file(merged, path)
    _write_export_config(resume_config, export_dir, step, current_window_size)
    return path
