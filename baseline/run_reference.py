"""Reference arm of the benchmark: the unmodified reference program, same metric and config.

`baseline/_ref/gpt_moe_reference/` is a verbatim copy of the reference's Python tree (it has neither
`setup.py` nor `pyproject.toml`, so `pip install --target baseline/_ref` refuses it; the copy is the install).
This harness drives it exactly the way its own `train.py` does (`train.py:37-236, 370-518`): NCCL process group,
`GPT(GPTConfig, TrainingConfig)`, `torch.compile` with the mode the config resolves to, `DistributedDataParallel`,
`configure_optimizers` (fused AdamW + its Muon), its `DataLoader` over `.npy` shards, pinned host-to-device copies,
autocast forward, backward with DDP gradient sync, token-scheduled LR, optimizer steps, `float(loss)` read-back.

What has to differ from the reference's stock configuration on this machine, and why:
* `linear_config`: every role `default` — its custom FP8 path refuses any GPU but capability (12, 0), and
  Transformer Engine / DeepGEMM are not installed (`model/linear/fp8/custom/dense.py:146-147`);
* third-party imports that need the network or a missing package (`tiktoken.get_encoding`, `transformer_engine`)
  are satisfied by the small stand-ins under `baseline/stubs/`;
* model/data shape: the benchmark's GPT-MoE-small config, on synthetic uniform token shards written at start-up.
"""
from __future__ import annotations

import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref", "gpt_moe_reference")


def _unavailable(reason: str) -> dict:
    return {"impl": "reference", "unavailable": reason.replace("\n", " ")[:300]}


def _write_shards(folder: str, tokens: int, vocab: int) -> None:
    import numpy as np
    os.makedirs(folder, exist_ok=True)
    rng = np.random.default_rng(0)
    for split, index in (("val", 0), ("train", 1)):
        path = os.path.join(folder, f"edufineweb_{split}_{index:06d}.npy")
        if not os.path.exists(path) or np.load(path, mmap_mode="r").shape[0] != tokens:
            np.save(path, rng.integers(0, vocab, tokens, dtype=np.uint16))


def run_reference(args) -> dict:
    if not os.path.isdir(REF):
        return _unavailable("baseline/_ref/gpt_moe_reference is missing (copy of the reference tree)")
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    sys.path.insert(0, os.path.join(HERE, "stubs"))
    sys.path.insert(0, REF)
    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP
    try:
        from config.model import GPTConfig
        from config.training import TrainingConfig
        from schedules.token import custom_schedule
        from model.gpt import GPT
        from optimizers.muon import Muon
        from data.loader import DataLoader
        from runtime.precision import configure_adamw_moments, precision_context
    except Exception as exc:  # import chain of the reference failed on this image
        return _unavailable(f"reference import failed: {type(exc).__name__}: {exc}")

    rank, local_rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29578")
    os.environ.setdefault("RANK", "0"); os.environ.setdefault("WORLD_SIZE", "1"); os.environ.setdefault("LOCAL_RANK", "0")
    device = f"cuda:{local_rank}"
    torch.cuda.set_device(device)
    dist.init_process_group(backend="nccl", device_id=local_rank)
    master = rank == 0

    batch, seq, window = 16, 2048, 1024
    tc = TrainingConfig()
    tc.gpu_batch_size_train = tc.gpu_batch_size_val = batch
    tc.seq_len_train = tc.seq_len_val = seq
    tc.max_seq_len = seq
    tc.total_tokens_per_step_train = world * batch * seq
    tc.batch_size_keys_schedule = {"fn": custom_schedule, "kwargs": {"values": [0]}}
    tc.batch_size_values_schedule = {"fn": custom_schedule, "kwargs": {"values": [batch]}}
    tc.swa_keys_schedule = {"fn": custom_schedule, "kwargs": {"values": [0]}}
    tc.swa_values_schedule = {"fn": custom_schedule, "kwargs": {"values": [window]}}
    for phase in tc.linear_config.values():
        for role in phase.values():
            role["precision"], role["backend"] = "default", "custom"
    tc.resolve(world)
    gc = GPTConfig(n_layers=12, hidden_size=768, mlp_hidden_dim=3072, use_tied_embeddings=False, n_heads=12, n_kv_heads=12,
                   attn_dim=768, rope_base_theta=10000, activation="swiglu", use_fair_swiglu=False, num_experts=8,
                   moe_top_k=1, use_qk_debug_log=False)

    torch.manual_seed(tc.base_seed + rank)
    torch.cuda.manual_seed(tc.base_seed + rank)
    torch.set_float32_matmul_precision(tc.float32_matmul_precision)
    raw = GPT(gc, tc)
    raw.to(device)
    mode = os.environ.get("REF_COMPILE_MODE", tc.torch_compile_mode)
    log = []
    data_dir = os.path.join(HERE, "_ref", "synthetic_shards")
    tokens_needed = world * batch * seq * (args.steps + args.warmup + 2) + 1
    if master:
        _write_shards(data_dir, tokens_needed, gc.vocab_size)
    dist.barrier()

    def build(compile_mode):
        model = raw if compile_mode == "eager" else torch.compile(raw, mode=compile_mode, fullgraph=tc.torch_compile_fullgraph,
                                                                  dynamic=tc.torch_compile_dynamic)
        return DDP(model, device_ids=[local_rank])

    optimizers = raw.configure_optimizers(tc.adamw_max_lr, tc.adamw_betas, tc.adamw_eps, tc.adamw_weight_decay, "cuda",
                                          muon_class=Muon, master_process=False, log_buffer=log)
    configure_adamw_moments(optimizers["adamw"], tc.use_bf16_adamw_moments)
    ctx = precision_context(tc, "cuda")
    loader = DataLoader(batch, seq, world, rank, data_dir, "train", pad_token_id=gc.pad_token_id, eos_token_id=gc.eos_token_id,
                        return_document_ids=raw.use_doc_masking, master_process=False, log_buffer=log)
    raw.sliding_window_size.fill_(window)
    spec = tc.lr_schedule[0]
    state = {"tokens": 0}

    def step(model):
        model.train()
        raw.set_precision_phase("training")
        for opt in optimizers.values():
            opt.zero_grad()
        losses = torch.zeros(3, device=device)
        x, y, docs = loader.next_batch()
        x = x.pin_memory().to(device, non_blocking=True)
        y = y.pin_memory().to(device, non_blocking=True)
        model.require_backward_grad_sync = True
        with ctx:
            loss, token_loss, balance = model(x, y, document_ids=docs)
        losses += torch.stack((loss.detach().float(), token_loss.detach().float(), balance.detach().float()))
        loss.backward()
        dist.all_reduce(losses, op=dist.ReduceOp.AVG)
        lr = spec["fn"](state["tokens"] - spec["start"], **spec["kwargs"])
        for group in optimizers["adamw"].param_groups:
            group["lr"] = lr
        for group in optimizers["muon"].param_groups:
            group["lr"] = lr * raw.muon_lr_scale
        raw.clear_fp8_weights()
        for opt in optimizers.values():
            opt.step()
        state["tokens"] += world * batch * seq
        return float(losses[0])

    model, used_mode, errors = None, None, []
    for candidate in dict.fromkeys([mode, "max-autotune-no-cudagraphs", "default", "eager"]):
        try:
            model = build(candidate)
            step(model)
            torch.cuda.synchronize()
            used_mode = candidate
            break
        except Exception as exc:
            errors.append(f"{candidate}: {type(exc).__name__}: {str(exc)[:120]}")
            torch._dynamo.reset()
            model = None
    if model is None:
        dist.destroy_process_group()
        return _unavailable("reference step failed in every compile mode: " + " | ".join(errors))
    for _ in range(max(0, args.warmup - 1)):
        step(model)

    dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    loss = None
    for _ in range(args.steps):
        loss = step(model)
    end.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    ms = torch.tensor([max(start.elapsed_time(end), wall_ms)], dtype=torch.float64, device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    dist.barrier()
    total_ms = float(ms.item())
    tokens = world * batch * seq * args.steps
    result = {
        "metric": "train tok/s (box, max over ranks)", "value": tokens / (total_ms / 1e3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"model": "GPT-MoE-small (12L d768 12x64 heads, SWA 1024, 8 SwiGLU experts h3072 top-1, vocab 50304)",
                   "global_batch": batch * world, "seq_len": seq, "parallelism": f"dp{world}",
                   "l2": "per-step working set >> 126 MB L2; no explicit flush"},
        "notes": {"torch_compile_mode": used_mode, "compile_fallbacks": errors, "linear_precision": "default (bf16 autocast)",
                  "optimizer": "the reference's Muon (Polar Express) + torch fused AdamW"},
        "e2e": {"value": tokens / (total_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * batch * seq * 8, "d2h_bytes_per_step": 4},
        "last_loss": loss,
    }
    dist.destroy_process_group()
    return result if master else {}
