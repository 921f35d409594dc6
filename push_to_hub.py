"""Upload a run's checkpoints and logs to a Hugging Face model repository.

The repository name encodes the GPU, batch size, sequence length, gradient-accumulation steps and, when the logs contain
them, the data-parallel world size, the final validation loss and the total training minutes — all parsed from the
run's own `config.txt` / `log.txt` (reference `push_to_hub.py:66-250`).  Needs network access and `hf_user` / `hf_token`.
"""
from __future__ import annotations

import argparse
import os
import re
import subprocess
from pathlib import Path
from typing import Optional

ROOT = Path(__file__).resolve().parent


def parse_run_metadata(timestamp: str, root: Path = ROOT) -> dict:
    folder = root / "configs_and_logs" / timestamp
    meta = {"ddp_world_size": None, "gpu_batch_size_train": None, "seq_len_train": None, "grad_accum_mini_steps": None,
            "val_loss": None, "total_train_time_min": None}
    config = folder / "config.txt"
    if config.exists():
        text = config.read_text(errors="ignore")
        for key in ("gpu_batch_size_train", "seq_len_train", "grad_accum_mini_steps"):
            m = re.search(rf"^{key}\s*[:=]\s*(\d+)\s*$", text, re.MULTILINE)
            if m:
                meta[key] = int(m.group(1))
    log = folder / "log.txt"
    if log.exists():
        text = log.read_text(errors="ignore")
        m = re.findall(r"^per-gpu gradient accumulation mini-steps:\s*(\d+)\s*$", text, re.MULTILINE)
        if m and meta["grad_accum_mini_steps"] is None:
            meta["grad_accum_mini_steps"] = int(m[-1])
        m = re.findall(r"total gpus:\s*(\d+)|over (\d+) gpus", text)
        if m:
            meta["ddp_world_size"] = int(next(x for x in m[-1] if x))
        m = re.findall(r"val loss:\s*([0-9]+(?:\.[0-9]+)?)", text)
        if m:
            meta["val_loss"] = float(m[-1])
        m = re.findall(r"total train time:\s*([0-9]+(?:\.[0-9]+)?)\s*min", text)
        if m:
            meta["total_train_time_min"] = float(m[-1])
    return meta


def gpu_name() -> str:
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=name", "--format=csv,noheader"], capture_output=True, text=True, timeout=20).stdout
        return re.sub(r"[^A-Za-z0-9]+", "-", out.strip().splitlines()[0]).strip("-") or "gpu"
    except Exception:
        return "gpu"


def build_repo_id(user: str, timestamp: str, meta: dict, gpu: Optional[str] = None) -> str:
    parts = ["nanogpt", gpu or gpu_name()]
    if meta["ddp_world_size"]:
        parts.append(f"x{meta['ddp_world_size']}")
    if meta["gpu_batch_size_train"]:
        parts.append(f"BS{meta['gpu_batch_size_train']}")
    if meta["seq_len_train"]:
        parts.append(f"SEQ{meta['seq_len_train']}")
    if meta["grad_accum_mini_steps"]:
        parts.append(f"GA{meta['grad_accum_mini_steps']}")
    if meta["val_loss"] is not None:
        parts.append(f"val{meta['val_loss']:.4f}")
    if meta["total_train_time_min"] is not None:
        parts.append(f"{meta['total_train_time_min']:.1f}min")
    parts.append(timestamp)
    return f"{user}/{'_'.join(parts)}"[:96]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--timestamp", required=True)
    ap.add_argument("--private", action="store_true")
    args = ap.parse_args()
    user = os.environ.get("hf_user") or os.environ.get("HF_USER")
    token = os.environ.get("hf_token") or os.environ.get("HF_TOKEN")
    if not user or not token:
        raise SystemExit("set hf_user and hf_token")
    from huggingface_hub import HfApi
    meta = parse_run_metadata(args.timestamp)
    repo_id = build_repo_id(user, args.timestamp, meta)
    api = HfApi(token=token)
    api.create_repo(repo_id, repo_type="model", private=args.private, exist_ok=True)
    for folder in ("checkpoints", "model_exports", "configs_and_logs"):
        path = ROOT / folder / args.timestamp
        if path.is_dir():
            api.upload_folder(repo_id=repo_id, repo_type="model", folder_path=str(path), path_in_repo=folder)
    print(f"uploaded to https://huggingface.co/{repo_id}")


if __name__ == "__main__":
    main()
