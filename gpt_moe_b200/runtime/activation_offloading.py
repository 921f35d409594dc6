"""CPU offloading of saved activations for the first N blocks.

While a block of the offloaded prefix runs forward, every large contiguous tensor that autograd saves
for backward is copied to pinned host memory on a side stream and its device storage is released;
in backward, the tensors of block i-1 are fetched back while block i's backward runs (one block of
prefetch), ordered by CUDA events.  Parameters, small tensors and non-contiguous tensors stay on the
device, and a storage saved more than once is copied once (reference
`runtime/activation_offloading.py:13-204`).  On CPU the hooks are inert.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
from torch import Tensor


class _Saved:
    """One offloaded activation: host copy, ready events and the lazily restored device tensor."""
    __slots__ = ("host", "device_tensor", "copied", "fetched", "shape", "dtype", "device")

    def __init__(self, tensor: Tensor, stream: torch.cuda.Stream) -> None:
        self.shape, self.dtype, self.device = tensor.shape, tensor.dtype, tensor.device
        self.host = torch.empty(tensor.shape, dtype=tensor.dtype, device="cpu", pin_memory=True)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            self.host.copy_(tensor, non_blocking=True)
            self.copied = torch.cuda.Event()
            self.copied.record(stream)
        tensor.record_stream(stream)          # the device buffer may be reused only after the copy has read it
        self.device_tensor: Optional[Tensor] = None
        self.fetched: Optional[torch.cuda.Event] = None

    def prefetch(self, stream: torch.cuda.Stream) -> None:
        if self.device_tensor is not None:
            return
        with torch.cuda.stream(stream):
            stream.wait_event(self.copied)
            self.device_tensor = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            self.device_tensor.copy_(self.host, non_blocking=True)
            self.fetched = torch.cuda.Event()
            self.fetched.record(stream)

    def get(self, stream: torch.cuda.Stream) -> Tensor:
        self.prefetch(stream)
        torch.cuda.current_stream().wait_event(self.fetched)
        self.device_tensor.record_stream(torch.cuda.current_stream())
        return self.device_tensor


class ActivationOffloading:
    def __init__(self, num_layers: int, min_bytes: int) -> None:
        self.num_layers, self.min_bytes = num_layers, min_bytes
        self.stream: Optional[torch.cuda.Stream] = None
        self.last_offloaded_bytes = 0
        self._groups: List[List[_Saved]] = []

    def _hooks(self, group: List[_Saved], params: set, seen: Dict[Tuple[int, int], _Saved]):
        def pack(t: Tensor):
            if (not t.is_cuda or t.data_ptr() in params or not t.is_contiguous()
                    or t.numel() * t.element_size() < self.min_bytes):
                return t
            key = (t.untyped_storage().data_ptr(), t.storage_offset())
            hit = seen.get(key)
            if hit is not None and hit.shape == t.shape and hit.dtype == t.dtype:
                return hit
            saved = _Saved(t, self.stream)
            seen[key] = saved
            group.append(saved)
            self.last_offloaded_bytes += t.numel() * t.element_size()
            return saved

        def unpack(obj):
            if not isinstance(obj, _Saved):
                return obj
            index = next((i for i, g in enumerate(self._groups) if obj in g), None)
            if index is not None and index > 0:          # fetch the previous block's activations one block ahead
                for other in self._groups[index - 1]:
                    other.prefetch(self.stream)
            return obj.get(self.stream)

        return pack, unpack

    def run(self, blocks, x: Tensor, ctx) -> Tuple[Tensor, Optional[Tensor]]:
        """Forward through all blocks, offloading what the first `num_layers` of them save."""
        balance = None
        if x.is_cuda and self.stream is None:
            self.stream = torch.cuda.Stream()
        self.last_offloaded_bytes = 0
        self._groups = []
        for i, block in enumerate(blocks):
            if x.is_cuda and i < self.num_layers:
                group: List[_Saved] = []
                self._groups.append(group)
                params = {p.data_ptr() for p in block.parameters()}
                pack, unpack = self._hooks(group, params, {})
                with torch.autograd.graph.saved_tensors_hooks(pack, unpack):
                    x, b = block(x, ctx)
            else:
                x, b = block(x, ctx)
            if b is not None:
                balance = b if balance is None else balance + b
        return x, balance
