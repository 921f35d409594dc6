"""Muon: momentum SGD whose 2-D updates are orthogonalised before being applied.

Update for a matrix W with gradient G (reference `optimizers/muon.py:147-224`):
    buf = momentum*buf + G ;  U = G + momentum*buf (Nesterov) or buf
    O = orthogonalise(U)   (Polar Express, quintic Newton-Schulz or SVD; fused (3d,d) matrices
                            are split into three squares first)
    W -= lr * sqrt(max(rows, cols)) * O
State key per parameter: `momentum_buffer` (full shape), as in the reference.

Sharding (new): with `owner_of` set by the engine, a rank updates only the matrices it owns;
the engine then all-gathers the updated weights.  The reference repeats the whole computation on
every rank.  On CUDA the momentum update, the Gram/Newton-Schulz GEMMs and the final
weight update run as hand-written kernels (`csrc/fused/loss_optim.cu`, `csrc/comm/fused_comm.cu`, the
tcgen05 GEMM in `csrc/gemm/gemm_bf16.cu` driven by `ops/cuda_ops.py::polar_express_bf16`); here is
the host orchestration and the CPU path.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, Optional

import torch
from torch import Tensor

from ..ops import reference as ref

zeropower_backends: Dict[str, Callable] = {
    "svd": lambda g, steps=None: ref.svd_orthogonalize(g),
    "newtonschulz5": lambda g, steps=5: ref.newton_schulz5(g, steps=steps),
    "polarexpress": lambda g, steps=5: ref.polar_express(g),
}


def _matrix_views(p: Tensor, g: Tensor, buf: Tensor):
    """Split a fused (3d, d) projection into three (d, d) problems (reference `muon.py:163-166`)."""
    if g.size(0) == 3 * g.size(1):
        d = g.size(1)
        return list(zip(p.split(d), g.split(d), buf.split(d)))
    return [(p, g, buf)]


class Muon(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 3e-4, momentum: float = 0.95, nesterov: bool = True,
                 backend: str = "newtonschulz5", backend_steps: int = 5) -> None:
        defaults = dict(lr=lr, momentum=momentum, nesterov=nesterov, backend=backend, backend_steps=backend_steps)
        super().__init__(params, defaults)
        self.owner_of: Optional[Callable[[Tensor], bool]] = None   # engine hook: does this rank own p?

    def _grad(self, p: Tensor) -> Optional[Tensor]:
        main = getattr(p, "main_grad", None)
        return main if main is not None else p.grad

    @torch.no_grad()
    def step(self, closure=None) -> None:
        for group in self.param_groups:
            lr, momentum, nesterov = group["lr"], group["momentum"], group["nesterov"]
            backend, steps = group["backend"], group["backend_steps"]
            work = []
            for p in group["params"]:
                g = self._grad(p)
                if g is None or (self.owner_of is not None and not self.owner_of(p)):
                    continue
                state = self.state[p]
                if "momentum_buffer" not in state:
                    state["momentum_buffer"] = torch.zeros_like(g)
                work.extend(_matrix_views(p.data, g, state["momentum_buffer"]))
            if not work:
                continue
            if work[0][0].is_cuda and backend == "polarexpress":
                from ..ops import cuda_ops
                cuda_ops.muon_polar_step(work, lr, momentum, nesterov)
                continue
            dtype = torch.bfloat16 if work[0][0].is_cuda else torch.float32
            for w, g, buf in work:
                buf.mul_(momentum).add_(g)
                update = g.add(buf, alpha=momentum) if nesterov else buf
                if backend == "polarexpress":
                    o = ref.polar_express(update, dtype=dtype)
                elif backend == "newtonschulz5":
                    o = ref.newton_schulz5(update, steps=steps, dtype=dtype)
                else:
                    o = ref.svd_orthogonalize(update)
                w.add_(o.to(w.dtype), alpha=-lr * max(w.shape) ** 0.5)
