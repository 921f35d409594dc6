"""Experiment runner: named experiments -> config overrides -> `torchrun train.py` -> optional Hub upload.

The reference runner (`experiments/run.py:14-166`) varies the program by applying patch files, trains, uploads and reverses
the patches, guarded by a repository lock and SIGTERM-safe process-group cleanup.  Here an experiment is a preset plus
`model.*` / `training.*` overrides (the capabilities the reference keeps in patches — MoE shape sweeps, MLA ranks, shared
expert — are ordinary config fields), so nothing has to be patched or reversed; the lock, the per-experiment console log,
the summary file, kill-the-whole-process-group on interrupt and upload-even-after-a-training-error behaviour are kept.
"""
from __future__ import annotations

import argparse
import fcntl
import os
import shlex
import signal
import subprocess
import sys
from datetime import datetime
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]

EXPERIMENTS = {
    "baseline": ("default", []),
    "small": ("small", []),
    "small-mxfp8": ("small", ["training.linear_config=mxfp8"]),
    "moe-8-top1": ("default", ["model.num_experts=8", "model.moe_top_k=1"]),
    "moe-16-top2": ("default", ["model.num_experts=16", "model.moe_top_k=2"]),
    "moe-16-top1": ("default", []),
    "moe-8-top1-wide": ("default", ["model.num_experts=8", "model.moe_top_k=1", "model.mlp_hidden_dim=4096"]),
    "moe-32-top2": ("default", ["model.num_experts=32", "model.moe_top_k=2"]),
    "moe-32-top1": ("default", ["model.num_experts=32", "model.moe_top_k=1"]),
    "moe-64-top1": ("default", ["model.num_experts=64", "model.moe_top_k=1"]),
    "mla-kv768": ("default", ["model.use_mla=True", "model.mla_kv_rank=768", "model.mla_qk_content_dim=48", "model.mla_qk_rope_dim=16"]),
    "mla-kv512": ("default", ["model.use_mla=True", "model.mla_kv_rank=512", "model.mla_qk_content_dim=48", "model.mla_qk_rope_dim=16"]),
    "mla-kv1024": ("default", ["model.use_mla=True", "model.mla_kv_rank=1024", "model.mla_qk_content_dim=48", "model.mla_qk_rope_dim=16"]),
    "moe-shared": ("default", ["model.moe_shared_expert_hidden_dim=2048"]),
    "wide-ep": ("wide_ep", []),
    "mla-ep": ("mla", []),
}


def run_command(command, log) -> int:
    """Run in its own process group; on any interruption terminate the whole group (SIGTERM, then SIGKILL after 30 s)."""
    log.write(f"\n$ {shlex.join(command)}\n")
    log.flush()
    process = subprocess.Popen(command, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
    try:
        return process.wait()
    except BaseException:
        if process.poll() is None:
            os.killpg(process.pid, signal.SIGTERM)
            try:
                process.wait(timeout=30)
            except subprocess.TimeoutExpired:
                os.killpg(process.pid, signal.SIGKILL)
                process.wait()
        raise


def _stop(signum, frame):
    raise SystemExit(128 + signum)


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description="Run named experiments: train, then upload to the Hub")
    parser.add_argument("experiments", nargs="*", metavar="NAME", help=f"experiment names in order (default: baseline); one of {', '.join(EXPERIMENTS)}")
    parser.add_argument("--nproc-per-node", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None, help="stop each run after this many steps")
    parser.add_argument("--no-upload", action="store_true")
    parser.add_argument("--dry-run", action="store_true", help="print the commands without running them")
    args = parser.parse_args(argv)
    unknown = [e for e in args.experiments if e not in EXPERIMENTS]
    if unknown:
        parser.error(f"unknown experiment(s) {unknown}; choose from: {', '.join(EXPERIMENTS)}")
    if args.nproc_per_node < 1:
        parser.error("--nproc-per-node must be positive")
    upload = not args.no_upload
    if upload and not args.dry_run:
        if not (os.environ.get("hf_user") or os.environ.get("HF_USER")) or not (os.environ.get("hf_token") or os.environ.get("HF_TOKEN")):
            parser.error("set hf_user/hf_token (or pass --no-upload) before starting")
    os.chdir(ROOT)
    signal.signal(signal.SIGTERM, _stop)
    batch = datetime.now().strftime("%Y%m%d_%H%M%S")
    runs_dir = ROOT / "configs_and_logs"
    runs_dir.mkdir(exist_ok=True)
    lock = (runs_dir / ".runner.lock").open("a")
    try:
        fcntl.flock(lock, fcntl.LOCK_EX | fcntl.LOCK_NB)
    except BlockingIOError:
        parser.error("another experiment runner is active in this repository")
    summary_path = ROOT / f"experiments-{batch}.log"
    failed = False
    with summary_path.open("x") as summary:
        summary.write("experiment\ttrain_exit\tupload_exit\ttimestamp\n")
        for index, name in enumerate(args.experiments or ["baseline"], 1):
            preset, overrides = EXPERIMENTS[name]
            stamp = datetime.now().strftime("%Y%m%d_%H%M%S")
            train = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
                     f"--nproc-per-node={args.nproc_per_node}", "train.py", "--preset", preset,
                     "--set", f"training.timestamp={stamp!r}"]
            for item in overrides:
                train += ["--set", item]
            if args.steps is not None:
                train += ["--steps", str(args.steps)]
            push = [sys.executable, "push_to_hub.py", "--timestamp", stamp]
            if args.dry_run:
                print(shlex.join(train))
                print(shlex.join(push))
                continue
            console = ROOT / f"experiment-{name}-{batch}-{index:02d}.log"
            print(f"experiment {name}; training output: {console}", flush=True)
            with console.open("x") as log:
                train_exit = run_command(train, log)
                upload_exit = run_command(push, log) if upload else 0      # a failed run still uploads its logs
            failed |= train_exit != 0 or upload_exit != 0
            summary.write(f"{name}\t{train_exit}\t{upload_exit}\t{stamp}\n")
            summary.flush()
    if args.dry_run:
        summary_path.unlink()
    return 1 if failed else 0


if __name__ == "__main__":
    raise SystemExit(main())
