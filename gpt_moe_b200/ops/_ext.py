"""Loader of the in-tree CUDA extension (`gpt_moe_b200/_C.so`).

The shared object is built by `csrc/build.py` (see `__graft_entry__.build`).  On import it is
rebuilt only if a source changed since the recorded stamp.  A missing or unloadable extension is
an error on any machine that has a GPU: there is no silent fallback for CUDA tensors.
"""
from __future__ import annotations

import importlib
import os

_ext = None


def load():
    global _ext
    if _ext is not None:
        return _ext
    from ..csrc import build as builder
    stamp = os.path.join(builder.BUILD, "stamp.txt")
    fresh = os.path.exists(builder.TARGET) and os.path.exists(stamp) and open(stamp).read() == builder.source_digest()
    if not fresh:
        builder.build()
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    # GM_CHECK_BOUNDS=1 selects the bounds-checked build of the same sources (`_C_checked.so`)
    _ext = importlib.import_module("gpt_moe_b200." + os.path.splitext(os.path.basename(builder.TARGET))[0])
    return _ext
