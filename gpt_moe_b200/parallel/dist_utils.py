"""Process-group helpers shared by the engines, the trainer and the evaluations."""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def env_rank_info():
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)))


def init_distributed(device_type: str, timeout_s: float = 600.0) -> None:
    """NCCL for GPUs, gloo for CPU runs; single-process runs get a world of one through a file-less TCP store."""
    if dist.is_initialized():
        return
    rank, local_rank, world = env_rank_info()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    kwargs = dict(rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    if device_type == "cuda":
        torch.cuda.set_device(local_rank)
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local_rank), **kwargs)
    else:
        dist.init_process_group(backend="gloo", **kwargs)


def is_dist() -> bool:
    return dist.is_available() and dist.is_initialized()


def world_size(group=None) -> int:
    return dist.get_world_size(group) if is_dist() else 1


def get_rank(group=None) -> int:
    return dist.get_rank(group) if is_dist() else 0


def barrier() -> None:
    if is_dist():
        dist.barrier()


def all_reduce(t: torch.Tensor, op=None, group=None) -> torch.Tensor:
    """In-place all-reduce; AVG is emulated as SUM / n so it also works on gloo."""
    if not is_dist() or world_size(group) == 1:
        return t
    if op == "avg":
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
        t /= world_size(group)
    else:
        dist.all_reduce(t, op=op or dist.ReduceOp.SUM, group=group)
    return t


def max_over_ranks(value: float, device) -> float:
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if is_dist() and world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
