"""Stand-alone GPU correctness script for the kernel families (counterpart of the reference's
`experiments/check_grouped.py`, `check_attention.py`, `check_qkv_norm_rope_fp8.py`): runs the GPU test modules that compare
every kernel with its plain-PyTorch definition — ragged and empty experts, widths that are not tile multiples,
non-contiguous inputs, top-k 1 and 2, attention windows — and prints one summary line.  Usage: `python experiments/check_kernels.py`.
"""
from __future__ import annotations

import os
import sys

import pytest

if __name__ == "__main__":
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.exit(pytest.main(["-q", "-m", "gpu", os.path.join(root, "tests", "test_gpu_ops.py"), os.path.join(root, "tests", "test_gpu_model.py")]))
