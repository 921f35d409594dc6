"""Per-kernel breakdown of one training step: `python -m gpt_moe_b200.utils.step_profile [--preset small] [--precision mxfp8|default] [--rows 40] [--set k=v ...]`.

Runs a few warm-up steps of the preset on synthetic data, records one step with `torch.profiler` (CUPTI kernel
timings, no replay) and prints the kernels sorted by total device time together with the step's wall time.  Shares of the
step are what to read off it; absolute kernel times under a profiler are slightly inflated.
"""
from __future__ import annotations

import argparse
import time

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="small")
    ap.add_argument("--rows", type=int, default=40)
    ap.add_argument("--precision", default="mxfp8", choices=["default", "mxfp8"])
    ap.add_argument("--set", dest="overrides", action="append", default=[])
    args = ap.parse_args()
    from torch.profiler import ProfilerActivity, profile
    from gpt_moe_b200.config import apply_overrides, get_preset
    from gpt_moe_b200.runtime.trainer import Trainer
    gpt_config, training_config = get_preset(args.preset, precision=args.precision)
    apply_overrides(gpt_config, training_config, args.overrides)
    training_config.kernel_warmup_train_steps = 0
    trainer = Trainer(gpt_config, training_config, device_type="cuda", quiet=True)
    for _ in range(3):
        trainer.train_step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        trainer.train_step()
        torch.cuda.synchronize()
    print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=args.rows, max_name_column_width=90))
    t0 = time.perf_counter()
    for _ in range(5):
        trainer.train_step(read_losses=False)
    torch.cuda.synchronize()
    print(f"step wall time without the profiler: {(time.perf_counter() - t0) / 5 * 1e3:.2f} ms")
    trainer.close()


if __name__ == "__main__":
    main()
