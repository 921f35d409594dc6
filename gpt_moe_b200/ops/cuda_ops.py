"""CUDA implementations of the ops in `api`, as autograd Functions over the sm_100a extension.

Conventions
* activations that feed GEMMs are bf16 and contiguous; the residual stream may be fp32;
* GEMM weights are bf16 "compute copies" of the fp32 master parameters.  A copy is refreshed when
  the parameter changes: optimizer kernels write through raw pointers, so they bump a global epoch
  (`mark_parameters_updated`) in addition to torch's own per-tensor version counter;
* a parameter with a `main_grad` attribute (set by the GPU engine) receives its weight gradient by
  direct accumulation from the GEMM epilogue and autograd gets `None` for it; otherwise the
  gradient is returned normally;
* every launch that can hit a bounded wait reports through the extension's status word;
  `check_status()` raises if any kernel gave up.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor

from . import _ext
from . import reference as ref

BF16 = torch.bfloat16


class _CountingExtension:
    """Proxy over the extension module that counts calls (every binding launches at least one kernel)."""

    def __init__(self, module) -> None:
        self._module = module
        self.calls = 0
        self._wrapped: dict = {}

    def __getattr__(self, name: str):
        fn = self._wrapped.get(name)
        if fn is None:
            target = getattr(self._module, name)

            launches = name not in ("read_status", "reset_status", "status_word_tensor", "read_bounds_status", "bounds_checked",
                                    "mla_decode_ok")     # bookkeeping calls launch nothing

            def fn(*args, _target=target, _launches=launches, **kwargs):
                self.calls += _launches
                return _target(*args, **kwargs)

            self._wrapped[name] = fn
        return fn


_proxy = None


def ext():
    global _proxy
    if _proxy is None:
        _proxy = _CountingExtension(_ext.load())
    return _proxy


_path_counts: dict = {}


def count_path(name: str) -> None:
    """Record that an op ran on path `name` (`attention:tcgen05`, `attention:sdpa`, `linear:torch`, ...)."""
    _path_counts[name] = _path_counts.get(name, 0) + 1


def path_counts() -> dict:
    """How often each op path ran in this process; a key that does not end in the kernel's own name is a library or torch path."""
    return dict(_path_counts)


def launch_count() -> int:
    """Number of extension launches issued so far by this process."""
    return ext().calls


def add_launches(count: int) -> None:
    """Account for kernels that ran without a Python call (a replayed CUDA graph): `count` = bindings recorded at capture."""
    ext().calls += int(count)


def check_status() -> None:
    code = ext().read_status()
    if code != 0:
        ext().reset_status()
        raise RuntimeError(f"a device-side bounded wait gave up (status {code}); the step is invalid")
    if ext().bounds_checked():                 # GM_CHECK_BOUNDS=1 build: a kernel met an out-of-range index and skipped the access
        code = ext().read_bounds_status()
        if code != 0:
            raise RuntimeError(f"bounds-checked build: a kernel skipped an out-of-range index (code {code})")
        changed = ext().verify_output_guards()      # GM_CANARIES=1: guard bytes around the bindings' allocations
        if changed != 0:
            raise RuntimeError(f"bounds-checked build: {changed} guard bytes around an output or scratch buffer were overwritten")


_status_host: dict = {}


def check_status_deferred() -> None:
    """`check_status` without a host synchronisation per call: the status word is copied to pinned host memory
    behind the work issued so far, and the copy made by the PREVIOUS call is examined (it has long completed in a
    training loop).  A step whose kernels gave up is therefore reported one call late; `check_status()` is the
    immediate form."""
    device = torch.cuda.current_device()
    slot = _status_host.get(device)
    if slot is None:
        slot = _status_host[device] = {"host": torch.zeros(1, dtype=torch.int32).pin_memory(), "event": None}
    if slot["event"] is not None:
        slot["event"].synchronize()
        code = int(slot["host"][0])
        if code != 0:
            slot["event"] = None
            ext().reset_status()
            raise RuntimeError(f"a device-side bounded wait gave up (status {code}); the step before this one is invalid")
    slot["host"].copy_(ext().status_word_tensor(), non_blocking=True)
    event = torch.cuda.Event()
    event.record()
    slot["event"] = event


# ---- compute copies of weights ---------------------------------------------------------------------------
_params_epoch = 0
_weight_cache: dict = {}


def mark_parameters_updated() -> None:
    global _params_epoch
    _params_epoch += 1


def clear_weight_cache() -> None:
    _weight_cache.clear()


def _cached(key, params: Sequence[Tensor], build):
    stamp = (_params_epoch,) + tuple(p._version for p in params)
    hit = _weight_cache.get(key)
    if hit is not None and hit[0] == stamp and all(a is b for a, b in zip(hit[1], params)):
        return hit[2]
    value = build(hit[2] if hit is not None else None)
    _weight_cache[key] = (stamp, tuple(params), value)
    return value


def _cast_into(src: Tensor, dst: Tensor) -> None:
    if src.dtype == torch.float32 and src.is_contiguous():
        ext().cast_bf16(src.detach(), dst)
    else:
        dst.copy_(src.detach())


def _compute_view(weights: Sequence[Tensor], stack: bool) -> Optional[Tensor]:
    """When an engine maintains bf16 copies (`param.compute`) laid out back to back, the concatenation / stack of
    the weights is simply a view of that memory."""
    copies = [getattr(w, "compute", None) for w in weights]
    if any(c is None for c in copies):
        return None
    first = copies[0]
    ptr = first.data_ptr()
    for c in copies:
        if c.data_ptr() != ptr or not c.is_contiguous():
            return None
        ptr += c.numel() * c.element_size()
    if stack:
        if any(c.shape != first.shape for c in copies):
            return None
        return torch.as_strided(first, (len(copies),) + tuple(first.shape), (first.numel(),) + tuple(first.stride()))
    rows = sum(c.shape[0] for c in copies)
    return torch.as_strided(first, (rows,) + tuple(first.shape[1:]), first.stride())


def bf16_weight(weights: Sequence[Tensor]) -> Tensor:
    """bf16 copy of `cat(weights, dim=0)` (one tensor: just its copy)."""
    if len(weights) == 1 and weights[0].dtype == BF16:
        return weights[0].detach()
    view = _compute_view(weights, stack=False)
    if view is not None:
        return view

    def build(old):
        rows = sum(w.shape[0] for w in weights)
        out = old if old is not None else torch.empty((rows,) + tuple(weights[0].shape[1:]), dtype=BF16, device=weights[0].device)
        r = 0
        for w in weights:
            _cast_into(w, out[r: r + w.shape[0]])
            r += w.shape[0]
        return out

    return _cached(("cat",) + tuple(id(w) for w in weights), weights, build)


def stacked_weight(weights: Sequence[Tensor]) -> Tensor:
    """bf16 [E, N, K] stack of same-shape expert weights."""
    view = _compute_view(weights, stack=True)
    if view is not None:
        return view

    def build(old):
        out = old if old is not None else torch.empty((len(weights),) + tuple(weights[0].shape), dtype=BF16, device=weights[0].device)
        for e, w in enumerate(weights):
            _cast_into(w, out[e])
        return out

    return _cached(("stack",) + tuple(id(w) for w in weights), weights, build)


def _as_bf16_2d(x: Tensor) -> Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.dtype != BF16:
        x2 = x2.to(BF16)
    return x2 if x2.is_contiguous() else x2.contiguous()


def _grad_targets(weights: Sequence[Tensor]) -> Optional[Tensor]:
    """If every weight has a `main_grad` and they are adjacent slices of one buffer, return that buffer view."""
    mains = [getattr(w, "main_grad", None) for w in weights]
    if any(m is None for m in mains):
        return None
    base = mains[0]
    ptr = base.data_ptr()
    for m in mains:
        if m.data_ptr() != ptr or not m.is_contiguous():
            return None
        ptr += m.numel() * m.element_size()
    rows = sum(m.shape[0] for m in mains)
    return torch.as_strided(base, (rows,) + tuple(base.shape[1:]), base.stride())


def _take_accumulate_flag(weights: Sequence[Tensor]) -> bool:
    """main_grad buffers are overwritten by the first micro-step's GEMM and accumulated into afterwards."""
    acc = all(getattr(w, "grad_ready", False) for w in weights)
    for w in weights:
        w.grad_ready = True
    return acc


# ---- linear -------------------------------------------------------------------------------------------------
class _LinearFn(torch.autograd.Function):
    """y = x @ cat(weights)^T in bf16 with fp32 accumulation; weight gradients in fp32."""

    @staticmethod
    def forward(ctx, x: Tensor, n_weights: int, *weights: Tensor) -> Tensor:
        x2 = _as_bf16_2d(x)
        w = bf16_weight(weights)
        y = torch.empty((x2.shape[0], w.shape[0]), dtype=BF16, device=x.device)
        ext().gemm_bf16(x2, w, y)
        ctx.save_for_backward(x2, w)
        ctx.weights = weights
        ctx.x_shape, ctx.x_dtype = x.shape, x.dtype
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy: Tensor):
        x2, w = ctx.saved_tensors
        weights = ctx.weights
        dy2 = _as_bf16_2d(dy)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x2)
            ext().gemm_bf16(dy2, w, dx, False, True)                    # dX = dY @ W   (W read MN-major)
            dx = dx.view(ctx.x_shape).to(ctx.x_dtype)
        grads: List[Optional[Tensor]] = [None] * len(weights)
        if any(ctx.needs_input_grad[2:]):
            target = _grad_targets(weights)
            if target is not None:
                ext().gemm_bf16(dy2, x2, target, True, True, 1.0, 0.0, None, _take_accumulate_flag(weights))
            else:
                dw = torch.empty((w.shape[0], w.shape[1]), dtype=torch.float32, device=w.device)
                ext().gemm_bf16(dy2, x2, dw, True, True)               # dW = dY^T @ X (both read MN-major)
                r = 0
                for i, p in enumerate(weights):
                    grads[i] = dw[r: r + p.shape[0]].to(p.dtype)
                    r += p.shape[0]
        return (dx, None) + tuple(grads)


def linear_multi(x: Tensor, weights: Sequence[Tensor], precision: str = "default") -> Tensor:
    if precision in ("mxfp8", "fp8"):
        from .mxfp8 import mxfp8_linear_multi
        return mxfp8_linear_multi(x, weights)
    return _LinearFn.apply(x, len(weights), *weights)


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor], precision: str = "default") -> Tensor:
    k, n = weight.shape[1], weight.shape[0]
    if k % 8 or n % 8 or n < 8:
        count_path("linear:torch")
        y = F.linear(x.to(BF16), weight.to(BF16))          # shapes TMA cannot address (row pitch not a multiple of 16 bytes)
    else:
        y = linear_multi(x, (weight,), precision)
    return y if bias is None else y + bias.to(y.dtype)


# ---- normalisation ----------------------------------------------------------------------------------------------
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Optional[Tensor], eps: float) -> Tensor:
        xc = x if x.is_contiguous() else x.contiguous()
        w = None if weight is None else weight.detach().float()
        y, rstd, _ = ext().rmsnorm_fwd(xc, w, eps)
        ctx.save_for_backward(xc, w if w is not None else torch.empty(0, device=x.device), rstd)
        ctx.has_weight = weight is not None
        ctx.weight_dtype = None if weight is None else weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):
        x, w, rstd = ctx.saved_tensors
        dy = dy if (dy.dtype == BF16 and dy.is_contiguous()) else dy.to(BF16).contiguous()
        dx, dw = ext().rmsnorm_bwd(dy, x, w if ctx.has_weight else None, rstd)
        return dx, (dw.to(ctx.weight_dtype) if ctx.has_weight else None), None


def rms_norm(x: Tensor, weight: Optional[Tensor], eps: float) -> Tensor:
    """bf16 output; fp32 or bf16 input; statistics fp32."""
    d = x.shape[-1]
    if x.dtype not in (torch.float32, BF16) or d % 128 or (d // 128) not in (1, 2, 4, 6, 8, 12, 16):
        count_path("rms_norm:torch")
        return ref.rms_norm(x, weight, eps).to(BF16)
    return _RMSNormFn.apply(x, weight, eps)


class _ResidualRMSNormFn(torch.autograd.Function):
    """x_new = x + beta * branch;  h = rmsnorm(x_new) * w.  One kernel forward; backward adds the norm's input
    gradient onto the residual gradient in the norm-backward kernel and derives d(branch), d(beta) in one more pass."""

    @staticmethod
    def forward(ctx, x: Tensor, branch: Tensor, beta: Tensor, weight: Tensor, eps: float, quantize: bool):
        xc = x if x.is_contiguous() else x.contiguous()
        br = branch if (branch.dtype == BF16 and branch.is_contiguous()) else branch.to(BF16).contiguous()
        w = weight.detach().float()
        b = beta.detach().float().reshape(1)
        res = ext().rmsnorm_fwd(xc, w, eps, br, None, b, quantize)
        h, rstd, x_new = res[0], res[1], res[2]
        ctx.save_for_backward(x_new, w, rstd, br, b)
        ctx.meta = (beta.shape, beta.dtype, weight.dtype, beta.requires_grad)
        if quantize:                           # the MXFP8 copy of h (payload, scale records) for the projection that consumes it
            ctx.mark_non_differentiable(res[3], res[4])
            return x_new, h, res[3], res[4]
        return x_new, h, None, None

    @staticmethod
    def backward(ctx, dx_new: Optional[Tensor], dh: Optional[Tensor], _dq=None, _dsf=None):
        x_new, w, rstd, br, b = ctx.saved_tensors
        beta_shape, beta_dtype, w_dtype, beta_grad = ctx.meta
        dw = None
        if dh is not None:
            dh = dh if (dh.dtype == BF16 and dh.is_contiguous()) else dh.to(BF16).contiguous()
            res = None if dx_new is None else (dx_new if dx_new.is_contiguous() else dx_new.contiguous())
            dxn, dw = ext().rmsnorm_bwd(dh, x_new, w, rstd, res)
            dw = dw.to(w_dtype)
        else:
            dxn = dx_new.contiguous()
        dbranch, dbeta = ext().residual_bwd(dxn, br, b)
        return dxn, dbranch, (dbeta.reshape(beta_shape).to(beta_dtype) if beta_grad else None), dw, None, None


def residual_rms_norm(x: Tensor, branch: Tensor, alpha: Optional[Tensor], beta: Optional[Tensor], weight: Tensor, eps: float,
                      quantize_out: bool = False):
    """(x_new, rmsnorm(x_new)) with x_new = alpha*x + beta*branch.  The fused kernel covers the common case
    (fp32 residual stream, no alpha); other cases compose the unfused ops.  `quantize_out`: the consumer of the normalised
    rows is an MXFP8 projection; the kernel then also writes their e4m3 payload and scale records, handed over as the
    attribute `mxq` of the returned tensor."""
    d = x.shape[-1]
    fused = (alpha is None and x.dtype == torch.float32 and weight is not None and d % 128 == 0
             and (d // 128) in (1, 2, 4, 6, 8, 12, 16) and x.numel() % 4 == 0)
    if not fused:
        x_new = (x if alpha is None else alpha * x) + (branch if beta is None else beta * branch)
        return x_new, rms_norm(x_new, weight, eps)
    if beta is None:
        beta = torch.ones(1, device=x.device)
    quantize = bool(quantize_out and d % 128 == 0)
    x_new, h, hq, hsf = _ResidualRMSNormFn.apply(x, branch, beta, weight, eps, quantize)
    if quantize:
        h.mxq = (hq, hsf)
    return x_new, h


class _SplitQKVFn(torch.autograd.Function):
    """Views of the packed projection output as q, k, v; the backward assembles one packed gradient instead of
    three zero-filled slice gradients."""

    @staticmethod
    def forward(ctx, qkv: Tensor, hq: int, hk: int, d: int):
        ctx.cfg = (hq, hk, d, qkv.shape)
        q = qkv[..., : hq * d].unflatten(-1, (hq, d))
        k = qkv[..., hq * d: (hq + hk) * d].unflatten(-1, (hk, d))
        v = qkv[..., (hq + hk) * d:].unflatten(-1, (hk, d))
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        hq, hk, d, shape = ctx.cfg
        # the attention kernel's backward hands over three views of one packed buffer: return that buffer as is
        if dq is not None and dk is not None and dv is not None and dq._base is not None and dq._base is dk._base and \
                dq._base is dv._base and dq._base.shape == shape and dq.storage_offset() == 0:
            return dq._base, None, None, None
        parts = []
        for g, h in ((dq, hq), (dk, hk), (dv, hk)):
            parts.append(g.flatten(-2) if g is not None else torch.zeros(shape[:-1] + (h * d,), dtype=BF16, device="cuda"))
        return torch.cat(parts, dim=-1), None, None, None


def split_qkv(qkv: Tensor, hq: int, hk: int, d: int):
    return _SplitQKVFn.apply(qkv, hq, hk, d)


# ---- RoPE + QK-norm ---------------------------------------------------------------------------------------------------
class _RopeQKNormFn(torch.autograd.Function):
    """Operates on the packed projection output qkv[tokens, (Hq + Hk + Hv) * D]; q and k heads are rotated and
    normalised, v passes through.  Output has the same packed layout."""

    @staticmethod
    def forward(ctx, qkv: Tensor, cos, sin, q_scale, k_scale, seq_len, hq, hk, d, eps, rms, smin, smax):
        out = torch.empty_like(qkv)
        qs = None if q_scale is None else q_scale.detach().float().reshape(-1).contiguous()
        ks = None if k_scale is None else k_scale.detach().float().reshape(-1).contiguous()
        # the kernel rotates / normalises the q and k heads and passes the remaining (value) columns through
        ext().rope_qknorm_fwd(qkv, out, cos, sin, qs, ks, seq_len, hq, hk, d, eps, rms, smin, smax, qkv.shape[-1] - (hq + hk) * d)
        ctx.save_for_backward(qkv, cos if cos is not None else qkv.new_empty(0), sin if sin is not None else qkv.new_empty(0),
                              qs if qs is not None else qkv.new_empty(0), ks if ks is not None else qkv.new_empty(0))
        ctx.cfg = (seq_len, hq, hk, d, eps, rms, smin, smax, cos is not None, q_scale is not None)
        ctx.scale_shapes = (None if q_scale is None else (q_scale.shape, q_scale.dtype),
                            None if k_scale is None else (k_scale.shape, k_scale.dtype))
        return out

    @staticmethod
    def backward(ctx, dout: Tensor):
        qkv, cos, sin, qs, ks = ctx.saved_tensors
        seq_len, hq, hk, d, eps, rms, smin, smax, has_rope, has_norm = ctx.cfg
        dout = dout if dout.is_contiguous() else dout.contiguous()
        dx = dout                             # in place: q and k columns are rewritten, v columns pass through unchanged
        (dscale,) = ext().rope_qknorm_bwd(qkv, dout, dx, cos if has_rope else None, sin if has_rope else None,
                                          qs if has_norm else None, ks if has_norm else None, seq_len, hq, hk, d, eps, rms, smin, smax)
        dq = dk = None
        if has_norm:
            (qshape, qdt), (kshape, kdt) = ctx.scale_shapes
            dq, dk = dscale[:hq].reshape(qshape).to(qdt), dscale[hq:].reshape(kshape).to(kdt)
        return dx, None, None, dq, dk, None, None, None, None, None, None, None, None


def rope_qk_norm_packed(qkv: Tensor, cos, sin, q_scale, k_scale, seq_len: int, hq: int, hk: int, d: int,
                        eps: float, rms: bool, smin: float, smax: float) -> Tensor:
    smin = max(smin, -3.0e38)
    smax = min(smax, 3.0e38)
    return _RopeQKNormFn.apply(qkv, cos, sin, q_scale, k_scale, seq_len, hq, hk, d, eps, rms, smin, smax)


class _RopeAttentionFn(torch.autograd.Function):
    """RoPE + QK-norm on the packed projection rows followed by causal (sliding-window) attention, as one autograd node:
    forward = rope kernel + attention forward kernel; backward = attention backward kernel, whose fp32 dQ accumulator is read
    directly by the rope backward kernel (no bf16 round trip of dQ), working in place on the packed gradient rows."""

    @staticmethod
    def forward(ctx, qkv: Tensor, cos, sin, q_scale, k_scale, batch, seq_len, hq, hk, d, eps, rms, smin, smax, window, scale, softcap, doc_start):
        c = ext()
        out = torch.empty_like(qkv)
        qs = None if q_scale is None else q_scale.detach().float().reshape(-1).contiguous()
        ks = None if k_scale is None else k_scale.detach().float().reshape(-1).contiguous()
        c.rope_qknorm_fwd(qkv, out, cos, sin, qs, ks, seq_len, hq, hk, d, eps, rms, smin, smax, qkv.shape[-1] - (hq + hk) * d)
        packed = out.view(batch, seq_len, -1)
        q = packed[..., : hq * d].unflatten(-1, (hq, d))
        k = packed[..., hq * d: (hq + hk) * d].unflatten(-1, (hk, d))
        v = packed[..., (hq + hk) * d:].unflatten(-1, (hk, d))
        o, lse = c.attn_fwd(q, k, v, window, scale, softcap, doc_start)
        ctx.doc_start = doc_start
        empty = qkv.new_empty(0)
        ctx.save_for_backward(qkv, out, o, lse, cos if cos is not None else empty, sin if sin is not None else empty,
                              qs if qs is not None else empty, ks if ks is not None else empty)
        ctx.cfg = (batch, seq_len, hq, hk, d, eps, rms, smin, smax, window, scale, softcap, cos is not None, q_scale is not None)
        ctx.scale_shapes = (None if q_scale is None else (q_scale.shape, q_scale.dtype),
                            None if k_scale is None else (k_scale.shape, k_scale.dtype))
        return o

    @staticmethod
    def backward(ctx, d_out: Tensor):
        c = ext()
        qkv, out, o, lse, cos, sin, qs, ks = ctx.saved_tensors
        batch, seq_len, hq, hk, d, eps, rms, smin, smax, window, scale, softcap, has_rope, has_norm = ctx.cfg
        packed = out.view(batch, seq_len, -1)
        q = packed[..., : hq * d].unflatten(-1, (hq, d))
        k = packed[..., hq * d: (hq + hk) * d].unflatten(-1, (hk, d))
        v = packed[..., (hq + hk) * d:].unflatten(-1, (hk, d))
        d_out = d_out if (d_out.dtype == BF16 and d_out.is_contiguous()) else d_out.to(BF16).contiguous()
        grad = torch.empty_like(packed)                               # dq columns are produced by the rope backward from the fp32 dQ
        dk = grad[..., hq * d: (hq + hk) * d].unflatten(-1, (hk, d))
        dv = grad[..., (hq + hk) * d:].unflatten(-1, (hk, d))
        dq32 = c.attn_bwd(q, k, v, o, d_out, lse, dk, dv, window, scale, softcap, ctx.doc_start)
        g2 = grad.view(batch * seq_len, -1)
        (dscale,) = c.rope_qknorm_bwd(qkv, g2, g2, cos if has_rope else None, sin if has_rope else None, qs if has_norm else None,
                                      ks if has_norm else None, seq_len, hq, hk, d, eps, rms, smin, smax, dq32.view(batch * seq_len, -1))
        dqs = dks = None
        if has_norm:
            (qshape, qdt), (kshape, kdt) = ctx.scale_shapes
            dqs, dks = dscale[:hq].reshape(qshape).to(qdt), dscale[hq:].reshape(kshape).to(kdt)
        return (g2, None, None, dqs, dks) + (None,) * 13


def rope_attention_packed(qkv: Tensor, cos, sin, q_scale, k_scale, batch: int, seq_len: int, hq: int, hk: int, d: int, eps: float,
                          rms: bool, smin: float, smax: float, window: Optional[int], scale: Optional[float], softcap: float = 0.0,
                          doc_start: Optional[Tensor] = None) -> Tensor:
    """qkv [batch * seq_len, (hq + 2 hk) * 64] bf16 -> attention output [batch, seq_len, hq, 64]."""
    smin = max(smin, -3.0e38)
    smax = min(smax, 3.0e38)
    w = seq_len if window is None else int(window)
    count_path("attention:tcgen05")
    return _RopeAttentionFn.apply(qkv, cos, sin, q_scale, k_scale, batch, seq_len, hq, hk, d, eps, rms, smin, smax, w,
                                  d ** -0.5 if scale is None else float(scale), float(softcap), doc_start)


def rope_qk_norm(q, k, cos, sin, q_scale, k_scale, eps, rms, scale_min, scale_max):
    """Unpacked entry (separate q and k tensors [B,T,H,D]): pack, run the fused kernel, unpack."""
    b, t, hq, d = q.shape
    hk = k.shape[2]
    if d not in (32, 64, 128) or hq + hk > 64:
        return ref.rope_qk_norm(q, k, cos, sin, q_scale, k_scale, eps, rms, scale_min, scale_max)
    packed = torch.cat((q.reshape(b * t, hq * d), k.reshape(b * t, hk * d)), dim=1).to(BF16)
    out = rope_qk_norm_packed(packed, None if cos is None else cos.float().contiguous(), None if sin is None else sin.float().contiguous(),
                              q_scale, k_scale, t, hq, hk, d, eps, rms, scale_min, scale_max)
    return out[:, : hq * d].reshape(b, t, hq, d), out[:, hq * d:].reshape(b, t, hk, d)


# ---- attention ---------------------------------------------------------------------------------------------------------
def attention(q, k, v, *, causal=True, window=None, scale=None, softcap_value=0.0, tanh_backend="exact",
              attn_mask=None, document_ids=None):
    from .attention_cuda import attention as impl
    return impl(q, k, v, causal=causal, window=window, scale=scale, softcap_value=softcap_value,
                tanh_backend=tanh_backend, attn_mask=attn_mask, document_ids=document_ids)


# ---- activation ------------------------------------------------------------------------------------------------------------
class _ActivationFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pre: Tensor, name: str) -> Tensor:
        pre = pre if (pre.dtype == BF16 and pre.is_contiguous()) else pre.to(BF16).contiguous()
        ctx.save_for_backward(pre)
        ctx.name = name
        return ext().activation_fwd(pre, name)[0]

    @staticmethod
    def backward(ctx, dact: Tensor):
        (pre,) = ctx.saved_tensors
        dact = dact if (dact.dtype == BF16 and dact.is_contiguous()) else dact.to(BF16).contiguous()
        return ext().activation_bwd(dact, pre, ctx.name)[0], None


def activate(x: Tensor, name: str) -> Tensor:
    width = x.shape[-1] // 2 if name == "swiglu" else x.shape[-1]
    if width % 8:                               # the kernels move 16-byte vectors
        return ref.activate(x, name)
    return _ActivationFn.apply(x, name)


# ---- router ---------------------------------------------------------------------------------------------------------------------
class _RouterFn(torch.autograd.Function):
    """fp32 softmax over the router logits, top-k, gate weights and the load-balance loss in one kernel (one more backward)."""

    @staticmethod
    def forward(ctx, logits: Tensor, top_k: int, renormalise: bool, want_balance: bool):
        lg = logits if logits.is_contiguous() else logits.contiguous()
        res = ext().router_fwd(lg, top_k, renormalise, want_balance)
        top_idx, gates = res[0], res[1]
        balance, counts = (res[2], res[3]) if want_balance else (None, None)
        ctx.save_for_backward(lg, top_idx, counts if counts is not None else lg.new_empty(0))
        ctx.cfg = (renormalise, want_balance)
        ctx.mark_non_differentiable(top_idx)
        return top_idx, gates, (balance.reshape(()) if want_balance else None)

    @staticmethod
    def backward(ctx, _didx, dgates: Optional[Tensor], dbalance: Optional[Tensor]):
        lg, top_idx, counts = ctx.saved_tensors
        renormalise, want_balance = ctx.cfg
        dg = None if dgates is None else dgates.float().contiguous()
        db = None if (dbalance is None or not want_balance) else dbalance.float().reshape(1).contiguous()
        if dg is None and db is None:
            return None, None, None, None
        return ext().router_bwd(lg, top_idx, dg, db, counts if db is not None else None, renormalise), None, None, None


def router(logits: Tensor, top_k: int, full_softmax: bool, want_balance: bool, num_experts: int):
    """(top_idx int64 [T, k], gates fp32 [T, k], balance loss or None) from router logits [T, E] (bf16 or fp32)."""
    if num_experts > 128 or top_k > 8 or logits.dtype not in (BF16, torch.float32):
        count_path("router:torch")
        top_idx, gates, probs = ref.router_gates(logits, top_k, full_softmax)
        return top_idx, gates, (ref.load_balance_loss(probs, top_idx, num_experts) if want_balance else None)
    renormalise = not (top_k == 1 or full_softmax)
    return _RouterFn.apply(logits, top_k, renormalise, want_balance)


# ---- mixture of experts -------------------------------------------------------------------------------------------------------
class _MoEExpertsFn(torch.autograd.Function):
    """route -> gather -> grouped up GEMM -> activation -> grouped down GEMM -> gated combine, with a hand-written backward."""

    @staticmethod
    def forward(ctx, hidden: Tensor, gates: Tensor, top_idx: Tensor, activation: str, num_experts: int, *weights: Tensor):
        c = ext()
        up, down = weights[:num_experts], weights[num_experts:]
        top_k = top_idx.shape[1]
        h2 = _as_bf16_2d(hidden)
        gates32 = gates.detach().float().contiguous()
        dest, src_of_row, seg_ends, counts, tile_expert, meta = c.route(top_idx.contiguous(), num_experts)
        (packed,) = c.gather_rows(h2, src_of_row, meta, top_k)
        w_up, w_down = stacked_weight(up), stacked_weight(down)
        cap = packed.shape[0]
        pre = torch.empty((cap, w_up.shape[1]), dtype=BF16, device=hidden.device)
        c.gemm_bf16(packed, w_up, pre, False, False, 1.0, 0.0, None, False, 1, tile_expert, meta, None)
        (act,) = c.activation_fwd(pre, activation, meta)
        y = torch.empty((cap, w_down.shape[1]), dtype=BF16, device=hidden.device)
        c.gemm_bf16(act, w_down, y, False, False, 1.0, 0.0, None, False, 1, tile_expert, meta, None)
        out = c.combine_fwd(y, dest, gates32)
        ctx.save_for_backward(packed, pre, act, y, dest, src_of_row, seg_ends, tile_expert, meta, gates32, w_up, w_down)
        ctx.activation, ctx.num_experts, ctx.weights = activation, num_experts, weights
        ctx.hidden_meta = (hidden.shape, hidden.dtype, gates.dtype)
        ctx.mark_non_differentiable(top_idx)
        return out.view(*hidden.shape[:-1], out.shape[-1]).to(hidden.dtype)

    @staticmethod
    def backward(ctx, dout: Tensor):
        c = ext()
        packed, pre, act, y, dest, src_of_row, seg_ends, tile_expert, meta, gates32, w_up, w_down = ctx.saved_tensors
        e = ctx.num_experts
        up, down = ctx.weights[:e], ctx.weights[e:]
        shape, dtype, gdtype = ctx.hidden_meta
        d2 = _as_bf16_2d(dout)
        dy, dgates = c.combine_bwd(d2, y, src_of_row, gates32, meta)
        dact = torch.empty_like(act)
        c.gemm_bf16(dy, w_down, dact, False, True, 1.0, 0.0, None, False, 1, tile_expert, meta, None)
        grads: List[Optional[Tensor]] = [None] * (2 * e)

        def wgrad(a: Tensor, b: Tensor, params: Sequence[Tensor], offset: int) -> None:
            target = _grad_targets(params)
            if target is not None:
                c.gemm_bf16(a, b, target.view(e, params[0].shape[0], params[0].shape[1]), True, True, 1.0, 0.0, None,
                            _take_accumulate_flag(params), 2, None, None, seg_ends)
                return
            dw = torch.empty((e, params[0].shape[0], params[0].shape[1]), dtype=torch.float32, device=a.device)
            c.gemm_bf16(a, b, dw, True, True, 1.0, 0.0, None, False, 2, None, None, seg_ends)
            for i, p in enumerate(params):
                grads[offset + i] = dw[i].to(p.dtype)

        wgrad(dy, act, down, e)
        (dpre,) = c.activation_bwd(dact, pre, ctx.activation, meta)
        wgrad(dpre, packed, up, 0)
        dhidden = None
        if ctx.needs_input_grad[0]:
            dpacked = torch.empty_like(packed)
            c.gemm_bf16(dpre, w_up, dpacked, False, True, 1.0, 0.0, None, False, 1, tile_expert, meta, None)
            dhidden = c.combine_fwd(dpacked, dest, None, gates32.shape[1]).view(shape).to(dtype)
        return (dhidden, dgates.to(gdtype), None, None, None) + tuple(grads)


def moe_experts(hidden, top_idx, gates, up_weights, down_weights, up_biases, down_biases, activation,
                up_precision, down_precision):
    if up_biases is not None or down_biases is not None:
        raise NotImplementedError("expert biases are supported on the CPU path only")
    if up_precision in ("mxfp8", "fp8") or down_precision in ("mxfp8", "fp8"):
        from .mxfp8 import mxfp8_moe_experts
        return mxfp8_moe_experts(hidden, top_idx, gates, up_weights, down_weights, activation)
    return _MoEExpertsFn.apply(hidden, gates, top_idx, activation, len(up_weights), *up_weights, *down_weights)


# ---- loss -----------------------------------------------------------------------------------------------------------------------
_loss_scale = 1.0


def set_loss_scale(scale: float) -> None:
    """Scale the training loop will apply to the loss before backward (1 / accumulation steps).  The fused
    LM-head loss computes its gradients during the forward pass and bakes this factor in."""
    global _loss_scale
    _loss_scale = float(scale)


class _LinearCrossEntropyFn(torch.autograd.Function):
    """mean CE of (x @ W^T) against targets without materialising all logits: rows are processed in chunks;
    each chunk's logits are overwritten in place by their gradient, which immediately feeds the dX and dW GEMMs."""

    CHUNK = 8192

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, targets: Tensor, ignore_index: int) -> Tensor:
        c = ext()
        x2 = _as_bf16_2d(x)
        w = bf16_weight((weight,))
        rows, vocab = x2.shape[0], w.shape[0]
        targets = targets.reshape(-1).contiguous()
        n_valid = (targets != ignore_index).sum().clamp_(min=1).float()
        need_grad = x.requires_grad or weight.requires_grad
        scale = (_loss_scale / n_valid).reshape(1)
        losses = torch.empty(rows, dtype=torch.float32, device=x.device)
        dx = torch.empty_like(x2) if need_grad else None
        dw = None
        target_buf = _grad_targets((weight,)) if need_grad else None
        accumulate = _take_accumulate_flag((weight,)) if target_buf is not None else False
        if need_grad and target_buf is None:
            dw = torch.empty(w.shape, dtype=torch.float32, device=x.device)
        chunk = min(_LinearCrossEntropyFn.CHUNK, rows)
        logits = torch.empty((chunk, vocab), dtype=BF16, device=x.device)
        for start in range(0, rows, chunk):
            n = min(chunk, rows - start)
            lg = logits[:n]
            xs = x2[start: start + n]
            c.gemm_bf16(xs, w, lg)
            losses[start: start + n] = c.ce_fwd_bwd(lg, targets[start: start + n], scale, ignore_index, need_grad)
            if need_grad:
                c.gemm_bf16(lg, w, dx[start: start + n], False, True)
                first = start == 0
                if target_buf is not None:
                    c.gemm_bf16(lg, xs, target_buf, True, True, 1.0, 0.0, None, accumulate or not first)
                else:
                    c.gemm_bf16(lg, xs, dw, True, True, 1.0, 0.0, None, not first)
        ctx.save_for_backward(dx if dx is not None else x2.new_empty(0), dw if dw is not None else x2.new_empty(0))
        ctx.meta = (x.shape, x.dtype, weight.dtype, _loss_scale)
        return losses.sum() / n_valid

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        dx, dw = ctx.saved_tensors
        x_shape, x_dtype, w_dtype, baked = ctx.meta
        ratio = grad_out / baked                      # 1 when the training loop applies the announced loss scale
        gx = (dx * ratio.to(dx.dtype)).view(x_shape).to(x_dtype) if dx.numel() else None
        gw = (dw * ratio).to(w_dtype) if dw.numel() else None
        return gx, gw, None, None


def linear_cross_entropy(x, weight, targets, ignore_index=-100):
    return _LinearCrossEntropyFn.apply(x, weight, targets, ignore_index)


def cross_entropy(logits, targets, ignore_index=-100):
    count_path("cross_entropy:torch")
    return ref.cross_entropy(logits, targets, ignore_index)


# ---- optimizers --------------------------------------------------------------------------------------------------------------------
def adamw_step(params, states, lr, beta1, beta2, eps, weight_decay) -> None:
    c = ext()
    for p, state in zip(params, states):
        grad = getattr(p, "main_grad", None)
        if grad is None:
            grad = p.grad
        step = state.get("_host_step")
        if step is None:                       # first step after construction or a checkpoint load
            step = int(round(float(state["step"])))
        step += 1
        state["_host_step"] = step             # the device tensor is refreshed lazily by AdamW.state_dict()
        if p.dtype != torch.float32 or not p.is_contiguous():
            raise ValueError("the CUDA AdamW kernel expects contiguous fp32 parameters")
        g = grad if (grad.dtype == torch.float32 and grad.is_contiguous()) else grad.float().contiguous()
        c.adamw(p.data, g, state["exp_avg"], state["exp_avg_sq"], getattr(p, "compute", None), lr, beta1, beta2, eps,
                weight_decay, step, 1.0)
    mark_parameters_updated()


_ptr_tables: dict = {}


def _ptr_table(tensors: Sequence[Tensor]) -> Tensor:
    key = tuple(t.data_ptr() for t in tensors)
    table = _ptr_tables.get(key)
    if table is None:
        if len(_ptr_tables) > 4096:
            _ptr_tables.clear()
        table = torch.tensor(key, dtype=torch.int64, device=tensors[0].device)
        _ptr_tables[key] = table
    return table


def polar_express_bf16(x: Tensor, sumsq: Optional[Tensor] = None) -> Tensor:
    """Five Polar Express iterations on a batch of wide bf16 matrices x[n, m, k] (m <= k), every product on the tcgen05 GEMM:
    A = X X^T; B = b A + c A A; X = a X + B X.  A and B are symmetric: their GEMMs compute the tiles on or above the
    diagonal and mirror them (reference optimizers/polar_express.py:60-121, :155-230).  x is pre-normalised, or `sumsq` holds
    the sum of squares of each matrix and the factor 1 / (1.02 * norm + 1e-6) is applied by the epilogues of the first
    iteration.  The buffer of x is reused as scratch from the second iteration on."""
    c = ext()
    n, m, k = x.shape
    a_buf = torch.empty((n, m, m), dtype=BF16, device=x.device)
    b_buf = torch.empty_like(a_buf)
    y = torch.empty_like(x)
    for step, (ca, cb, cc) in enumerate(ref.POLAR_EXPRESS_COEFFS):
        first = sumsq if step == 0 else None
        c.gemm_bf16(x, x, a_buf, symmetric=True, batch_sumsq=first, scale_mode=2 if first is not None else 0)      # A = X X^T
        c.gemm_bf16(a_buf, a_buf, b_buf, False, False, cc, cb, a_buf, symmetric=True)                               # B = c A A^T + b A
        c.gemm_bf16(b_buf, x, y, False, True, 1.0, ca, x, batch_sumsq=first, scale_mode=1 if first is not None else 0)   # Y = B X + a X
        x, y = y, x
    return x


def muon_polar_step(work: List[Tuple[Tensor, Tensor, Tensor]], lr: float, momentum: float, nesterov: bool,
                    max_batch: int = 128) -> None:
    """work: (weight fp32, gradient fp32, momentum buffer fp32) triples, all 2-D.  Same-shape matrices are
    processed together: momentum/Nesterov/bf16 pack (transposed when tall) -> normalise -> Polar Express ->
    W += -lr * sqrt(max(rows, cols)) * O."""
    c = ext()
    buckets: dict = {}
    for w, g, buf in work:
        buckets.setdefault((tuple(w.shape), w.stride(0), g.stride(0), buf.stride(0)), []).append((w, g, buf))
    for (shape, ws, gs, bs), items in buckets.items():
        rows, cols = shape
        small = min(rows, cols) < 8 or rows % 8 or cols % 8       # rows the kernels cannot address as 16-byte pieces
        for start in range(0, len(items), max_batch):
            batch = items[start: start + max_batch]
            n = len(batch)
            alpha = -lr * max(rows, cols) ** 0.5
            if small:        # e.g. a router with an odd expert count
                for w, g, buf in batch:
                    buf.mul_(momentum).add_(g)
                grads = torch.stack([g.add(buf, alpha=momentum) if nesterov else buf for _, g, buf in batch])
                o = ref.polar_express(grads)
                for (w, _, _), oi in zip(batch, o):
                    w.add_(oi.to(w.dtype), alpha=alpha)
                continue
            tall = rows > cols
            m, k = (cols, rows) if tall else (rows, cols)
            packed = torch.empty((n, m, k), dtype=BF16, device=batch[0][0].device)
            sumsq = torch.zeros(n, dtype=torch.float32, device=packed.device)
            c.muon_prepare(_ptr_table([g for _, g, _ in batch]), _ptr_table([b for _, _, b in batch]), packed, sumsq,
                           rows, cols, gs, bs, momentum, nesterov, tall, 1.0)
            o = polar_express_bf16(packed)
            compute = [getattr(w, "compute", None) for w, _, _ in batch]
            bf16_ptrs = _ptr_table(compute) if all(t is not None for t in compute) else None
            c.muon_apply(_ptr_table([w for w, _, _ in batch]), bf16_ptrs, o, rows, cols, ws, alpha, tall)
    mark_parameters_updated()
