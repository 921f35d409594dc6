"""Failure detection without touching a GPU: host watchdog, a rank that never joins, a corrupted checkpoint,
a loader that raises, and the experiment runner's process-group cleanup."""
import os
import subprocess
import sys
import time

import pytest
import torch

from dist_helpers import free_port


def test_watchdog_fires_after_deadline_and_not_when_disarmed():
    from gpt_moe_b200.runtime.watchdog import StepWatchdog
    fired = []
    dog = StepWatchdog(0.15, on_timeout=fired.append, poll_s=0.02)
    dog.arm(); time.sleep(0.05); dog.disarm(); time.sleep(0.3)
    assert not fired and not dog.fired
    dog.arm(); time.sleep(0.5)
    assert len(fired) == 1 and fired[0] > 0.15 and dog.fired
    dog.stop()


def _lonely_rank(port):
    """A 2-rank job whose second rank never starts: rendezvous must fail within the timeout instead of hanging."""
    import datetime
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    t0 = time.time()
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        dist.barrier()
    except Exception as exc:
        print(f"DETECTED {type(exc).__name__} after {time.time() - t0:.1f}s")
        return
    print("NOT DETECTED")


def test_missing_rank_is_detected_by_timeout():
    code = f"import sys; sys.path.insert(0, {os.path.dirname(__file__)!r}); from test_failure_detection import _lonely_rank; _lonely_rank({free_port()})"
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert "DETECTED" in out.stdout and "NOT DETECTED" not in out.stdout, out.stdout + out.stderr


def _dying_peer(rank, world):
    """Rank 1 leaves between steps; rank 0's next collective must raise instead of blocking forever."""
    import datetime
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    t = torch.ones(1)
    dist.all_reduce(t)                      # step 1 completes on both ranks
    if rank == 1:
        os._exit(0)                         # leaves with nothing in flight
    time.sleep(0.5)
    try:
        dist.all_reduce(t)
        return "no error"
    except Exception as exc:
        return f"raised {type(exc).__name__}"


def test_peer_exit_between_steps_raises_on_survivor(tmp_path):
    import torch.multiprocessing as mp
    from dist_helpers import _entry
    port = free_port()
    ctx = mp.spawn(_entry, args=(2, port, _dying_peer, str(tmp_path), ()), nprocs=2, join=False)
    deadline = time.time() + 60
    while time.time() < deadline and not os.path.exists(os.path.join(str(tmp_path), "result_0.pt")):
        time.sleep(0.2)
        try:
            ctx.join(timeout=0.1)
        except Exception:
            pass
    result = torch.load(os.path.join(str(tmp_path), "result_0.pt"), weights_only=False)
    assert result.startswith("raised"), result


def test_corrupted_training_state_is_rejected(tmp_path):
    from gpt_moe_b200.checkpointing import checkpoint as ckpt
    from gpt_moe_b200.config import build_resume_config, get_preset
    gc, tc = get_preset("tiny_cpu")
    tc.resolve(1)
    bad = tmp_path / "training_state_step_0000001.pt"
    bad.write_bytes(b"not a checkpoint")
    weights = tmp_path / "model_step_0000001_val_na_train_1.0000.safetensors"
    weights.write_bytes(b"")
    tc.resume_checkpoint_path, tc.resume_state_dict_path = str(weights), str(bad)
    with pytest.raises(Exception):
        ckpt.load_checkpoint(tc, gc, 0, 1, build_resume_config(gc, tc))
    torch.save({"format_version": 1}, bad)
    with pytest.raises(ValueError, match="format version 2"):
        ckpt.load_checkpoint(tc, gc, 0, 1, build_resume_config(gc, tc))


def test_loader_failure_surfaces_from_train_step():
    from gpt_moe_b200.config import get_preset
    from gpt_moe_b200.runtime.trainer import Trainer
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()), RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
    gc, tc = get_preset("tiny_cpu")
    gc.n_layers, gc.vocab_size = 1, 512
    tc.kernel_warmup_train_steps = 0
    trainer = Trainer(gc, tc, device_type="cpu", quiet=True)

    class Broken:
        def next_batch(self):
            raise OSError("shard vanished")

    trainer.train_data_loader = Broken()
    with pytest.raises(OSError, match="shard vanished"):
        trainer.train_step()
    trainer.close()


def test_runner_terminates_the_process_group_on_interrupt(tmp_path):
    """SIGTERM to the runner while a training command is running: the child's whole process group is terminated."""
    import signal
    experiments = os.path.join(os.path.dirname(os.path.dirname(__file__)), "experiments")
    marker = tmp_path / "child.pid"
    child = f"import os, time; open({str(marker)!r}, 'w').write(str(os.getpid())); time.sleep(600)"
    driver = (f"import sys, signal; sys.path.insert(0, {experiments!r}); import run as runner\n"
              f"signal.signal(signal.SIGTERM, runner._stop)\n"
              f"log = open({str(tmp_path / 'log.txt')!r}, 'w')\n"
              f"runner.run_command([sys.executable, '-c', {child!r}], log)\n")
    proc = subprocess.Popen([sys.executable, "-c", driver])
    deadline = time.time() + 30
    while not (marker.exists() and marker.read_text()) and time.time() < deadline:
        time.sleep(0.05)
    pid = int(marker.read_text())
    os.kill(pid, 0)                                   # the child is alive
    proc.send_signal(signal.SIGTERM)
    assert proc.wait(timeout=60) == 128 + signal.SIGTERM
    time.sleep(0.3)
    with pytest.raises(ProcessLookupError):
        os.kill(pid, 0)                               # terminated together with its process group


def test_runner_dry_run_lists_commands(capsys):
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(__file__)), "experiments"))
    import run as runner
    assert runner.main(["moe-32-top2", "mla-kv512", "--dry-run", "--nproc-per-node", "2", "--no-upload"]) == 0
    out = capsys.readouterr().out
    assert "model.num_experts=32" in out and "model.use_mla=True" in out and "--nproc-per-node=2" in out
