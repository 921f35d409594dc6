"""Spawn helpers for the multi-process CPU (gloo) tests."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, out_dir, args):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    torch.set_num_threads(2)
    try:
        result = fn(rank, world, *args)
        torch.save(result, os.path.join(out_dir, f"result_{rank}.pt"))
    except Exception:
        with open(os.path.join(out_dir, f"error_{rank}.txt"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(fn, world, out_dir, *args, join_timeout=240):
    """Run fn(rank, world, *args) in `world` processes; returns the list of their results."""
    port = free_port()
    ctx = mp.spawn(_entry, args=(world, port, fn, str(out_dir), args), nprocs=world, join=False)
    import time
    deadline, ok = time.time() + join_timeout, False
    while time.time() < deadline:
        if ctx.join(timeout=5):         # True once every process has been joined
            ok = True
            break
    if not ok:
        for p in ctx.processes:
            if p.is_alive():
                p.terminate()
    errors = [open(os.path.join(out_dir, f)).read() for f in sorted(os.listdir(out_dir)) if f.startswith("error_")]
    assert not errors, "\n".join(errors)
    assert ok, "ranks did not finish in time"
    return [torch.load(os.path.join(out_dir, f"result_{r}.pt"), weights_only=False) for r in range(world)]
