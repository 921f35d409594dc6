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
    module = importlib.import_module("gpt_moe_b200." + os.path.splitext(os.path.basename(builder.TARGET))[0])
    if module.bounds_checked() and module.output_guards_enabled():
        module = _SynchronisingProxy(module)
    _ext = module
    return _ext


class _SynchronisingProxy:
    """Debugging aid of the bounds-checked build with GM_CANARIES=1: every call into the extension is followed by a device
    synchronisation, so an asynchronous launch or execution error is raised by the call that caused it rather than by a later one."""

    def __init__(self, module):
        self._module = module

    def __getattr__(self, name):
        attr = getattr(self._module, name)
        if not callable(attr) or name in ("read_status", "reset_status", "bounds_checked", "output_guards_enabled", "verify_output_guards",
                                          "read_bounds_status", "status_word_tensor"):
            return attr

        def call(*args, **kwargs):
            import torch
            result = attr(*args, **kwargs)
            if torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing():
                torch.cuda.synchronize()
            return result

        call.__name__ = name
        return call
