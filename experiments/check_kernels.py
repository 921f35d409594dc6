"""Stand-alone GPU correctness script for the kernel families (counterpart of the reference's
`experiments/check_grouped.py`, `check_attention.py`, `check_qkv_norm_rope_fp8.py`): runs the GPU test modules that compare
every kernel with its plain-PyTorch definition — ragged and empty experts, widths that are not tile multiples,
non-contiguous inputs, gradients requested for a subset of the inputs or outputs, quantised weights cached across
accumulation micro-steps, top-k 1 and 2, attention windows, MXFP8 against its emulation — first on the normal build and
then on the bounds-checked build (`GM_CHECK_BOUNDS=1`, every data-dependent index tested), then on the same build with
`GM_CANARIES=1` (guard bytes around every output and scratch buffer the bindings allocate, a device synchronisation after every
call), and prints one summary line per pass.  Usage: `python experiments/check_kernels.py [--skip-checked]`.
"""
from __future__ import annotations

import os
import sys

import pytest

if __name__ == "__main__":
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = [os.path.join(root, "tests", name) for name in ("test_gpu_ops.py", "test_gpu_mxfp8.py", "test_gpu_model.py")]
    code = pytest.main(["-q", "-m", "gpu"] + files)
    if code == 0 and "--skip-checked" not in sys.argv:
        # the extension variant is chosen when it is first loaded: the checked pass runs in a fresh interpreter
        env = dict(os.environ, GM_CHECK_BOUNDS="1")
        code = subprocess.run([sys.executable, "-m", "pytest", "-q", "-m", "gpu"] + files[:2], env=env, cwd=root).returncode
        if code == 0:
            env["GM_CANARIES"] = "1"
            code = subprocess.run([sys.executable, "-m", "pytest", "-q", "-m", "gpu"] + files[:2], env=env, cwd=root).returncode
    sys.exit(code)
