"""Host-side step watchdog.

The reference has no failure detection: a rank that dies leaves the others blocked in a
collective until NCCL's own timeout (`train.py:747-758`).  `StepWatchdog` is a daemon thread
armed at the start of every step; if the step does not finish within `deadline_s` it calls
`on_timeout` (default: print a diagnostic, abort the process group and exit with status 75) so a
launcher can restart the job from the last checkpoint.  Nothing here touches the GPU.
"""
from __future__ import annotations

import os
import sys
import threading
import time
from typing import Callable, Optional


def _default_abort(elapsed: float) -> None:
    sys.stderr.write(f"[watchdog] step exceeded its deadline ({elapsed:.1f} s); aborting for restart from checkpoint\n")
    sys.stderr.flush()
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.distributed_c10d._abort_process_group() if hasattr(dist.distributed_c10d, "_abort_process_group") else None
    except Exception:
        pass
    os._exit(75)


class StepWatchdog:
    def __init__(self, deadline_s: float, on_timeout: Optional[Callable[[float], None]] = None, poll_s: float = 0.05) -> None:
        self.deadline_s = deadline_s
        self.on_timeout = on_timeout or _default_abort
        self.poll_s = poll_s
        self._armed_at: Optional[float] = None
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self.fired = False
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def arm(self) -> None:
        with self._lock:
            self._armed_at = time.monotonic()

    def disarm(self) -> None:
        with self._lock:
            self._armed_at = None

    def stop(self) -> None:
        self._stop.set()

    def _loop(self) -> None:
        while not self._stop.wait(self.poll_s):
            with self._lock:
                armed = self._armed_at
            if armed is not None and time.monotonic() - armed > self.deadline_s:
                self.fired = True
                with self._lock:
                    self._armed_at = None
                self.on_timeout(time.monotonic() - armed)
