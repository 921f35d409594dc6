"""Headline benchmark: training throughput (tokens/s, whole job) of GPT-MoE-small on N B200s.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run)
    python bench.py --impl reference --gpus N ...            the unmodified reference through its own code path

Config (named in the JSON line): 12 layers, d_model 768, 12 heads x 64, QK-RMSNorm + RoPE, sliding-window
causal attention (window 1024) over 2048 tokens, 8 SwiGLU experts (hidden 3072) top-1, vocab 50304,
micro-batch 16 x 2048 tokens per GPU, Muon (Polar Express) + AdamW, bf16 activations with the QKV / output / expert
projections in MXFP8 (e4m3, 32-element E8M0 blocks; `--precision default` runs them in bf16 too), synthetic uniform token
ids from seed 0, random normal(0, 0.02) weights.  Weak scaling: per-GPU work is fixed.

Two measurements, both after W warm-up steps, both max over ranks:
  value : K optimizer steps with inputs already on the device, timed with CUDA events;
  e2e   : K optimizer steps through `Trainer.train_step()` — each step copies its token batch from pinned host
          memory to the device and reads the step's loss back to the host.
One step touches several GB of activations and weights, far more than the 126 MB L2, so no explicit flush is
needed between timed iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import threading
import time

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi every 200 ms while the timed region runs."""

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self) -> None:
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks = sorted(float(r[1]) for r in self.rows if r[1].replace(".", "").isdigit())
        reasons = set()
        for r in self.rows:
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": float(self.rows[0][2]) if self.rows else None,
                "samples": len(clocks), "reasons": sorted(reasons)}


MODEL_NAMES = {
    "small": "GPT-MoE-small (12L d768 12x64 heads, SWA 1024, 8 SwiGLU experts h3072 top-1, vocab 50304)",
    "wide_ep": "GPT-MoE-wide (12L d768 12x64 heads, SWA 1024, 32 SwiGLU experts h1536 top-2, expert parallel, vocab 50304)",
    "mla": "GPT-MoE-MLA (24L d1024 16 heads, MLA kv rank 512 + rope 64, 64 routed SwiGLU experts h1024 top-1 + shared h2048, expert parallel, vocab 50304)",
}


def run_ours(args) -> dict:
    import torch
    from gpt_moe_b200.config import apply_overrides, get_preset
    from gpt_moe_b200.ops import cuda_ops
    from gpt_moe_b200.parallel import dist_utils as du
    from gpt_moe_b200.runtime.trainer import Trainer

    gpt_config, training_config = get_preset(args.preset, precision=args.precision)
    apply_overrides(gpt_config, training_config, args.overrides)
    training_config.kernel_warmup_train_steps = 0
    trainer = Trainer(gpt_config, training_config, device_type="cuda", quiet=True)
    world, rank = trainer.world_size, trainer.rank
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    cfg = training_config
    tokens_per_step = cfg.gpu_batch_size_train * cfg.seq_len_train * world * cfg.grad_accum_mini_steps

    for _ in range(args.warmup):
        trainer.train_step()
    torch.cuda.synchronize()

    # device-resident inputs for the kernel-only measurement
    gen = torch.Generator().manual_seed(1234 + rank)
    staged = []
    for _ in range(max(1, min(args.steps, 4))):
        ids = torch.randint(0, gpt_config.vocab_size, (cfg.gpu_batch_size_train, cfg.seq_len_train + 1), generator=gen)
        staged.append((ids[:, :-1].contiguous().to(trainer.device), ids[:, 1:].contiguous().to(trainer.device), None))

    sampler = ClockSampler(trainer.local_rank)
    if rank == 0:
        sampler.start()

    def timed(step_fn) -> float:
        du.barrier()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(args.steps):
            step_fn(i)
        end.record()
        torch.cuda.synchronize()
        du.barrier()
        return du.max_over_ranks(start.elapsed_time(end), trainer.device)

    launches_before = cuda_ops.launch_count()
    device_ms = timed(lambda i: trainer.train_step([staged[i % len(staged)]] * cfg.grad_accum_mini_steps, read_losses=False))
    launches = cuda_ops.launch_count() - launches_before

    losses = []
    wall0 = time.perf_counter()
    e2e_ms = timed(lambda i: losses.append(trainer.train_step()["loss"]))
    wall_ms = du.max_over_ranks((time.perf_counter() - wall0) * 1e3, trainer.device)
    e2e_ms = max(e2e_ms, wall_ms)
    clocks = sampler.stop() if rank == 0 else {}
    cuda_ops.check_status()

    # exposed communication: the same steps with every peer offset pointing at local memory and without barriers
    # (same arithmetic and bytes, nothing crosses NVLink); the difference to the normal step time is what communication adds
    exposed_ms = None
    if world > 1 and hasattr(trainer.engine, "set_comm_dry_run") and trainer.ep_size == 1:
        trainer.engine.set_comm_dry_run(True)
        for _ in range(4):                    # enough for the engine to capture the graph of the dry step before timing starts
            trainer.train_step([staged[0]] * cfg.grad_accum_mini_steps, read_losses=False)
        dry_ms = timed(lambda i: trainer.train_step([staged[i % len(staged)]] * cfg.grad_accum_mini_steps, read_losses=False))
        trainer.engine.set_comm_dry_run(False)
        exposed_ms = (device_ms - dry_ms) / args.steps

    engine_info = trainer.engine.describe() if hasattr(trainer.engine, "describe") else {"engine": type(trainer.engine).__name__}
    result = {
        "metric": "train tok/s (box, max over ranks)", "value": tokens_per_step * args.steps / (device_ms / 1e3),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": device_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.precision == "default" else "bf16+mxfp8", "data": "synthetic",
        "config": {"model": MODEL_NAMES.get(args.preset, args.preset),
                   "global_batch": cfg.gpu_batch_size_train * world, "seq_len": cfg.seq_len_train,
                   "parallelism": f"dp{world}" + (f"+ep{trainer.ep_size}" if trainer.ep_size > 1 else ""),
                   "l2": "per-step working set >> 126 MB L2; no explicit flush"},
        "notes": {"optimizer": "muon(polar express)+adamw", "linear_precision": args.precision, **engine_info,
                  "op_paths": cuda_ops.path_counts()},
        "clocks": clocks,
        "e2e": {"value": tokens_per_step * args.steps / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": 2 * cfg.gpu_batch_size_train * cfg.seq_len_train * 8 * cfg.grad_accum_mini_steps,
                "d2h_bytes_per_step": 12, "last_loss": losses[-1] if losses else None},
        "gpu_launches": launches, "impl": "gpt_moe_b200", "exposed_comm_ms_per_step": exposed_ms,
    }
    trainer.close()
    return result if rank == 0 else {}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="mxfp8", choices=["default", "mxfp8"],
                    help="mxfp8 (default): QKV / output / expert projections run MXFP8 forward and input-gradient GEMMs, as the benchmark "
                         "configuration names them; default: every GEMM in bf16")
    ap.add_argument("--preset", default="small", choices=["small", "wide_ep", "mla"],
                    help="small is the headline configuration; wide_ep and mla are the expert-parallel configurations (ours only)")
    ap.add_argument("--set", dest="overrides", action="append", default=[])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        from baseline.run_reference import run_reference
        result = run_reference(args)
    else:
        result = run_ours(args)
    if result:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
