"""Rotary position tables.

fp32 cos/sin tables [max_seq_len, head_size/2] held as non-persistent buffers, i.e. never written
to checkpoints (reference `model/position/rotary.py:10-41`).  Rotation itself is interleaved-pair
RoPE and lives in `ops` because it is fused with QK-norm on the GPU.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.reference import rope_tables


class Rotary(nn.Module):
    def __init__(self, head_size: int, base_theta: float, max_seq_len: int) -> None:
        super().__init__()
        assert head_size % 2 == 0, "RoPE needs an even head size"
        inv_freq = 1.0 / (base_theta ** (torch.arange(0, head_size, 2, dtype=torch.float32) / head_size))
        cos, sin = rope_tables(head_size, base_theta, max_seq_len)
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self.register_buffer("cos_cached", cos, persistent=False)
        self.register_buffer("sin_cached", sin, persistent=False)
