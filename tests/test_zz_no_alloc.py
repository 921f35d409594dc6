"""The allocation-free `gm_residual_bwd_noalloc` entry point, called through its exported C symbol.

Some hosts of this library may not allocate device memory (their memory pool belongs to someone else, or they are
inside a stream capture), so this variant keeps its scratch in a fixed array inside the library.  The test checks it
against the regular (allocating) binding on two calls in a row — the second call reuses the scratch the first one left
behind.  Collected last so that a `-x` run has already executed every other test.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    import gpt_moe_b200
    from gpt_moe_b200.ops import _ext
    _ext.load()                       # builds the extension if needed and loads libtorch first
    lib = ctypes.CDLL(os.path.join(os.path.dirname(gpt_moe_b200.__file__), "_C.so"))
    fn = lib.gm_residual_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p]
    return fn


def test_no_alloc_entry_point_matches_allocating_binding():
    from gpt_moe_b200.ops import cuda_ops
    fn = _library()
    torch.manual_seed(0)
    for n, beta_value in ((4096 * 768, 0.37), (1024 * 256, -1.5)):        # two calls in a row, different sizes
        dxn = torch.randn(n, device="cuda")
        branch = torch.randn(n, device="cuda").bfloat16()
        beta = torch.tensor([beta_value], device="cuda")
        want_dbranch, want_dbeta = cuda_ops.ext().residual_bwd(dxn, branch, beta)
        dbranch = torch.empty_like(branch)
        dbeta = torch.full((1,), float("nan"), device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        stream = torch.cuda.current_stream().cuda_stream
        rc = fn(dxn.data_ptr(), branch.data_ptr(), beta.data_ptr(), dbranch.data_ptr(), dbeta.data_ptr(), n, stream)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.memory_allocated() == before            # nothing was allocated through torch
        assert torch.equal(dbranch, want_dbranch)
        rel = abs(dbeta.item() - want_dbeta.item()) / (abs(want_dbeta.item()) + 1e-6)
        assert rel < 1e-5, (dbeta.item(), want_dbeta.item())
        exact = (dxn.double() * branch.double()).sum().item()
        assert abs(dbeta.item() - exact) / (abs(exact) + 1e-6) < 6e-3


def test_no_alloc_entry_point_rejects_bad_sizes():
    fn = _library()
    x = torch.zeros(8, device="cuda")
    b = torch.zeros(8, device="cuda", dtype=torch.bfloat16)
    one = torch.ones(1, device="cuda")
    args = (x.data_ptr(), b.data_ptr(), one.data_ptr(), b.data_ptr(), one.data_ptr())
    assert fn(*args, 6, None) == 1                      # not a multiple of 4
    assert fn(*args, 0, None) == 1
    assert fn(*args, (1 << 34) + 4, None) == 1          # beyond the stated maximum
    assert fn(None, b.data_ptr(), one.data_ptr(), b.data_ptr(), one.data_ptr(), 8, None) == 1
