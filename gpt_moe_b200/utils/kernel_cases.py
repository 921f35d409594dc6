"""Run one hot kernel on a small, fixed case: `python -m gpt_moe_b200.utils.kernel_cases <case> [--iters N]`.

Meant for profiling (`ncu -k regex:<kernel> ... python -m gpt_moe_b200.utils.kernel_cases <case>`) and for quick timing
with CUDA events.  Cases are larger than the 126 MB L2 where DRAM traffic matters and hold at most a few GB.
"""
from __future__ import annotations

import argparse

import torch


def _timed(fn, iters):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "gemm_mxfp8", "quantize", "gemm_wgrad", "grouped", "attn_fwd", "attn_fwd_full", "attn_bwd", "attn_bwd_full", "rs_muon", "ce", "rmsnorm", "rope", "rope_bwd", "ep_dispatch", "ep_combine", "rmsnorm_bwd", "attn_fwd_mla", "attn_bwd_mla", "gemm_xxt", "gemm_xxt_full", "polar", "gemm_big", "gemm_mxfp8_big", "gemm_mxfp8_down", "quantize_weight", "mma_issue"])
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--single-tile", action="store_true", help="attention: the basic kernels (one query tile per CTA forward, unpipelined backward)")
    args = ap.parse_args()
    from gpt_moe_b200.ops import attention_tc, cuda_ops
    c = cuda_ops.ext()
    dev = "cuda"
    torch.manual_seed(0)
    if args.case == "mma_issue":                 # device clocks of chained tcgen05.mma instructions, one CTA (csrc/bench/mma_issue.cu)
        names = ["M128 N128", "M128 N256", "M128 N64", "M128 N16", "M128 N64, A in TMEM, B MN-major", "M128 N256, A in TMEM",
                 "M64 N256, A MN-major", "M64 N128, A MN-major"]
        for shape, name in enumerate(names):
            issue, done = c.mma_issue_bench(shape, 64)
            print(f"mma_issue: {name}: 64 instructions issued in {issue} clk, complete after {done} clk = {done / 64:.1f} clk each")
        return
    flops = bytes_ = 0
    if args.case == "gemm":                      # QKV projection shape: [32768, 768] x [2304, 768]^T
        a = torch.randn(32768, 768, device=dev).bfloat16(); b = torch.randn(2304, 768, device=dev).bfloat16()
        d = torch.empty(32768, 2304, device=dev, dtype=torch.bfloat16)
        fn = lambda: c.gemm_bf16(a, b, d)
        flops = 2 * 32768 * 2304 * 768
    elif args.case == "gemm_mxfp8":              # same shape on e4m3 operands with 32-element UE8M0 block scales
        a = torch.randn(32768, 768, device=dev).bfloat16(); b = torch.randn(2304, 768, device=dev).bfloat16()
        aq, asf = c.mxfp8_quantize(a); bq, bsf = c.mxfp8_quantize(b)
        d = torch.empty(32768, 2304, device=dev, dtype=torch.bfloat16)
        fn = lambda: c.gemm_mxfp8(aq, asf, bq, bsf, d)
        flops = 2 * 32768 * 2304 * 768
    elif args.case in ("gemm_big", "gemm_mxfp8_big"):   # long contraction: the main loop dominates, the epilogue is amortised over 64 K blocks
        a = torch.randn(8192, 8192, device=dev).bfloat16(); b = torch.randn(8192, 8192, device=dev).bfloat16()
        d = torch.empty(8192, 8192, device=dev, dtype=torch.bfloat16)
        if args.case == "gemm_big":
            fn = lambda: c.gemm_bf16(a, b, d)
        else:
            aq, asf = c.mxfp8_quantize(a); bq, bsf = c.mxfp8_quantize(b)
            fn = lambda: c.gemm_mxfp8(aq, asf, bq, bsf, d)
        flops = 2 * 8192 ** 3
    elif args.case == "gemm_mxfp8_down":         # expert down-projection shape: [32768, 3072] x [768, 3072]^T
        a = torch.randn(32768, 3072, device=dev).bfloat16(); b = torch.randn(768, 3072, device=dev).bfloat16()
        aq, asf = c.mxfp8_quantize(a); bq, bsf = c.mxfp8_quantize(b)
        d = torch.empty(32768, 768, device=dev, dtype=torch.bfloat16)
        fn = lambda: c.gemm_mxfp8(aq, asf, bq, bsf, d)
        flops = 2 * 32768 * 768 * 3072
    elif args.case == "quantize_weight":         # both quantised layouts of 96 expert up-projection weights in one pass
        w = torch.randn(96, 6144, 768, device=dev).bfloat16()
        fn = lambda: c.mxfp8_quantize_weight(w)
        bytes_ = 96 * 6144 * 768 * 4 + 2 * 96 * 6144 * 768 // 32
    elif args.case == "quantize":                # bf16 -> e4m3 + scale records, 256 MB in
        a = torch.randn(65536, 2048, device=dev).bfloat16()
        fn = lambda: c.mxfp8_quantize(a)
        bytes_ = 65536 * 2048 * 3 + 65536 * 2048 // 32
    elif args.case == "gemm_wgrad":              # dW = dY^T X, both operands MN-major, fp32 output, split-K
        dy = torch.randn(32768, 2304, device=dev).bfloat16(); x = torch.randn(32768, 768, device=dev).bfloat16()
        dw = torch.empty(2304, 768, device=dev)
        fn = lambda: c.gemm_bf16(dy, x, dw, True, True)
        flops = 2 * 32768 * 2304 * 768
    elif args.case == "grouped":                 # expert up-projection: 8 experts, 32768 routed rows
        idx = torch.randint(0, 8, (32768, 1), device=dev)
        dest, src, seg, counts, tiles, meta = c.route(idx, 8)
        hidden = torch.randn(32768, 768, device=dev).bfloat16()
        (packed,) = c.gather_rows(hidden, src, meta, 1)
        w = torch.randn(8, 6144, 768, device=dev).bfloat16()
        out = torch.empty(packed.shape[0], 6144, device=dev, dtype=torch.bfloat16)
        fn = lambda: c.gemm_bf16(packed, w, out, False, False, 1.0, 0.0, None, False, 1, tiles, meta, None)
        flops = 2 * 32768 * 6144 * 768
    elif args.case in ("attn_fwd", "attn_fwd_full", "attn_bwd", "attn_bwd_full"):  # 4 (full: 16) x 2048 tokens, 12 heads, window 1024
        b_, t, h, d = (16 if args.case.endswith("_full") else 4), 2048, 12, 64
        packed = torch.randn(b_, t, 3 * h * d, device=dev).bfloat16().requires_grad_()
        q, k, v = cuda_ops.split_qkv(packed, h, h, d)
        keys = sum(min(i, 1024) + 1 for i in range(t))
        if not args.case.startswith("attn_bwd"):
            fn = lambda: c.attn_fwd(q.detach(), k.detach(), v.detach(), 1024, d ** -0.5, single_tile=args.single_tile)
            flops = 4 * d * keys * b_ * h
        else:                                        # the binding itself: delta pre-pass, zeroed fp32 dQ, the backward kernel
            qd, kd, vd = q.detach(), k.detach(), v.detach()
            out, lse = c.attn_fwd(qd, kd, vd, 1024, d ** -0.5)
            g = torch.randn_like(out)
            dk, dv = torch.empty_like(kd), torch.empty_like(vd)
            fn = lambda: c.attn_bwd(qd, kd, vd, out, g, lse, dk, dv, 1024, d ** -0.5, 0.0, None, args.single_tile)
            flops = 10 * d * keys * b_ * h
    elif args.case in ("attn_fwd_mla", "attn_bwd_mla"):   # multi-head latent attention shape: 128-wide query/key heads, 64-wide values, causal 4096
        b_, t, h = 2, 4096, 16
        q = torch.randn(b_, t, h, 128, device=dev).mul_(0.5).bfloat16().requires_grad_()
        k = torch.randn(b_, t, h, 128, device=dev).mul_(0.5).bfloat16().requires_grad_()
        v = torch.randn(b_, t, h, 64, device=dev).bfloat16().requires_grad_()
        pairs = t * (t + 1) // 2 * b_ * h
        if args.case == "attn_fwd_mla":
            fn = lambda: c.attn_fwd(q.detach(), k.detach(), v.detach(), t, 128 ** -0.5)
            flops = 2 * (128 + 64) * pairs
        else:
            out = attention_tc.attention(q, k, v, window=None, scale=None)
            g = torch.randn_like(out)
            fn = lambda: torch.autograd.grad(out, (q, k, v), g, retain_graph=True)
            flops = 2 * (128 + 64 + 64 + 128 + 128) * pairs
    elif args.case in ("gemm_xxt", "gemm_xxt_full"):   # A = X X^T for 96 expert up-projection gradients [768, 6144]; triangle-and-mirror or every tile
        x = torch.randn(96, 768, 6144, device=dev).mul_(0.01).bfloat16()
        a = torch.empty(96, 768, 768, device=dev, dtype=torch.bfloat16)
        fn = lambda: c.gemm_bf16(x, x, a, symmetric=args.case == "gemm_xxt")
        flops = 2 * 96 * 768 * 768 * 6144                 # of the full product: the symmetric form does two thirds of it
    elif args.case == "polar":                   # five Polar Express iterations on the same batch
        x = torch.randn(96, 768, 6144, device=dev)
        x = (x / (x.norm(dim=(-2, -1), keepdim=True) * 1.02 + 1e-6)).bfloat16()
        fn = lambda: cuda_ops.polar_express_bf16(x)
        flops = 5 * 96 * (4 * 768 * 768 * 6144 + 2 * 768 ** 3)
    elif args.case == "rs_muon":                 # reduce + momentum + pack for 16 matrices of 6144 x 768 (world of one)
        grads = [torch.randn(6144, 768, device=dev) for _ in range(16)]
        bufs = [torch.zeros(6144, 768, device=dev) for _ in range(16)]
        packed = torch.empty(16, 768, 6144, device=dev, dtype=torch.bfloat16)
        sumsq = torch.zeros(16, device=dev)
        gp, bp = cuda_ops._ptr_table(grads), cuda_ops._ptr_table(bufs)
        fn = lambda: c.rs_muon_prepare(gp, bp, packed, sumsq, 6144, 768, 768, 768, 0.95, True, True, [0])
        bytes_ = 16 * 6144 * 768 * (4 + 4 + 4 + 2 + 2 + 2)
    elif args.case == "ce":
        logits = torch.randn(4096, 50304, device=dev).bfloat16()
        targets = torch.randint(0, 50304, (4096,), device=dev)
        scale = torch.ones(1, device=dev)
        fn = lambda: c.ce_fwd_bwd(logits, targets, scale, -100, True)
        bytes_ = 4096 * 50304 * 2 * 3
    elif args.case == "rmsnorm_bwd":            # backward of the fused residual + RMSNorm: fp32 residual stream, bf16 dy, residual gradient added
        x = torch.randn(32768, 768, device=dev); dy = torch.randn(32768, 768, device=dev).bfloat16()
        w = torch.ones(768, device=dev); rstd = torch.ones(32768, device=dev); res = torch.randn(32768, 768, device=dev)
        fn = lambda: c.rmsnorm_bwd(dy, x, w, rstd, res)
        bytes_ = 32768 * 768 * 14
    elif args.case in ("rope", "rope_bwd"):     # packed QKV rows of 32768 tokens: 12 q + 12 k heads rotated and normalised, 12 v heads passed through
        qkv = torch.randn(32768, 2304, device=dev).bfloat16()
        out = torch.empty_like(qkv)
        pos = torch.arange(2048, device=dev).float()[:, None] * (10000.0 ** (-torch.arange(32, device=dev).float() / 32))[None, :]
        cos, sin = pos.cos().contiguous(), pos.sin().contiguous()
        qs, ks = torch.ones(12, device=dev), torch.ones(12, device=dev)
        if args.case == "rope":
            fn = lambda: c.rope_qknorm_fwd(qkv, out, cos, sin, qs, ks, 2048, 12, 12, 64, 1e-6, True, -3e38, 5.0, 768)
            bytes_ = 32768 * 2304 * 2 * 2
        else:
            dy = torch.randn_like(qkv)
            fn = lambda: c.rope_qknorm_bwd(qkv, dy, dy, cos, sin, qs, ks, 2048, 12, 12, 64, 1e-6, True, -3e38, 5.0)
            bytes_ = 32768 * 1536 * 2 * 3
    elif args.case in ("ep_dispatch", "ep_combine"):   # group of one: every row takes the peer-memory path with a zero offset
        tokens, d, experts = 32768, 768, 8
        idx = torch.randint(0, experts, (tokens, 1), device=dev)
        hidden = torch.randn(tokens, d, device=dev).bfloat16()
        dest, _, local_ends, counts, _, _ = c.route(idx, experts)
        table = torch.zeros(experts, dtype=torch.int32, device=dev)
        c.ep_push_counts(counts, table, [0], 0)
        cap = tokens + experts * 256
        my_base, seg_ends, valid_ends, tiles, meta = c.ep_plan(table, 1, 0, experts, cap)
        recv = torch.zeros(cap, d, device=dev, dtype=torch.bfloat16)
        (route_row,) = c.ep_dispatch(hidden, idx, dest, local_ends, my_base, None, None, recv, [0], experts)
        gates = torch.ones(tokens, 1, device=dev)
        if args.case == "ep_dispatch":
            fn = lambda: c.ep_dispatch(hidden, idx, dest, local_ends, my_base, None, None, recv, [0], experts)
        else:
            fn = lambda: c.ep_combine(recv, idx, route_row, gates, False, [0], experts)
        bytes_ = tokens * d * 2 * 2
    else:
        x = torch.randn(32768, 768, device=dev)
        w = torch.ones(768, device=dev)
        fn = lambda: c.rmsnorm_fwd(x, w, 1e-6)
        bytes_ = 32768 * 768 * 6
    ms = _timed(fn, args.iters)
    cuda_ops.check_status()
    rate = f"{flops / ms / 1e9:.1f} TFLOP/s" if flops else f"{bytes_ / ms / 1e6:.1f} GB/s"
    print(f"{args.case}: {ms * 1e3:.1f} us per call, {rate}")


if __name__ == "__main__":
    main()
