"""GPU data-parallel engine.

`build_cuda_engine` returns the engine used on CUDA devices.  It keeps the `HostEngine`
interface (forward_backward / step / zero_grad / checkpoint helpers).
"""
from __future__ import annotations

from .ddp_engine import HostEngine


class CudaHostEngine(HostEngine):
    """NCCL collectives + this framework's kernels for everything on-device: the measured NCCL baseline."""

    def forward_backward(self, model, x, y, document_ids, loss_scale: float, last_micro_step: bool):
        from ..ops import cuda_ops
        cuda_ops.set_loss_scale(loss_scale)
        return super().forward_backward(model, x, y, document_ids, loss_scale, last_micro_step)

    def step(self) -> None:
        from ..ops import cuda_ops
        super().step()
        cuda_ops.mark_parameters_updated()
        cuda_ops.check_status()


def build_cuda_engine(model, training_config, optimizers, ep_size: int = 1, ep_group=None):
    return CudaHostEngine(model, training_config, optimizers, dp_group=None, ep_size=ep_size)
