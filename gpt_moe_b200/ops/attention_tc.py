"""Front end of the tcgen05 attention kernels (`csrc/attention`)."""
from __future__ import annotations

from typing import Optional

from torch import Tensor


def supported(q: Tensor, k: Tensor, v: Tensor, softcap_value: float) -> bool:
    return False


def attention(q: Tensor, k: Tensor, v: Tensor, *, window: Optional[int], scale: Optional[float]) -> Tensor:
    raise NotImplementedError
