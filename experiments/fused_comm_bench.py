"""Microbenchmarks of the fused compute+collective kernels against the same math done with NCCL calls.

Run with one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        experiments/fused_comm_bench.py [--part rs|ag|ep|all] [--quick] [--out results.json]

Parts
  rs   gradient reduce-scatter + Muon momentum / Nesterov / bf16 pack / Frobenius norm.
       fused: `rs_muon_prepare` sums the owner's matrices straight out of every rank's gradient buffer.
       nccl : `reduce_scatter_tensor` of the flat fp32 bucket, then the local `muon_prepare` kernel.
  ag   Muon apply + parameter all-gather.
       fused: `muon_apply_push` updates the fp32 master and stores the bf16 copy into every rank's weight buffer.
       nccl : local `muon_apply`, bf16 cast, `all_gather_into_tensor`.
  ep   expert-parallel MoE layer forward+backward (dispatch, grouped SwiGLU GEMMs, combine), Zipf(1.1) routing.
       fused: rows stored to / loaded from the owners' buffers by the dispatch / combine kernels.
       nccl : counted `all_to_all_single` exchanges around the same grouped GEMM kernels.
Every number is device time (CUDA events), max over ranks, after warm-up; inputs exceed the L2 for all but the smallest
buckets.  The roofline of a case is the slower of FLOPs / measured GEMM peak and NVLink bytes per GPU / 770 GB/s.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

LINK_GBS = 770.0           # measured peer copy bandwidth per direction per GPU
GEMM_TFLOPS = 1683.1       # measured cuBLAS bf16 burst


def timed(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    t = torch.tensor([start.elapsed_time(end) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def bench_rs_ag(args, results):
    from gpt_moe_b200.ops import cuda_ops
    from gpt_moe_b200.parallel.fused_engine import PeerBarrier, SymmetricBuffer
    c = cuda_ops.ext()
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    barrier = PeerBarrier(dev)                   # the engine's bounded device-side barrier: it is part of what the fused arm costs
    rows, cols = 768, 768
    sizes_mb = [1, 16, 256] if args.quick else [1, 4, 16, 64, 256, 1024]
    for mb in sizes_mb:
        per_mat = rows * cols
        n_mats = max(world, (mb << 20) // 4 // per_mat // world * world)        # matrices in the bucket (fp32 gradient bytes = mb)
        mine = n_mats // world
        numel = n_mats * per_mat
        grads = SymmetricBuffer(numel, torch.float32, dev)
        shadow = SymmetricBuffer(numel, torch.bfloat16, dev)          # bf16 wire format: peers read this copy of the gradients
        weights = SymmetricBuffer(numel, torch.bfloat16, dev)
        grads.tensor.normal_(0, 1e-3)
        lo = rank * mine
        my_grads = [grads.tensor[(lo + i) * per_mat: (lo + i + 1) * per_mat].view(rows, cols) for i in range(mine)]
        bufs = [torch.zeros(rows, cols, device=dev) for _ in range(mine)]
        masters = [torch.randn(rows, cols, device=dev) for _ in range(mine)]
        my_w = [weights.tensor[(lo + i) * per_mat: (lo + i + 1) * per_mat].view(rows, cols) for i in range(mine)]
        packed = torch.empty(mine, rows, cols, dtype=torch.bfloat16, device=dev)
        sumsq = torch.zeros(mine, device=dev)
        gp, bp = cuda_ops._ptr_table(my_grads), cuda_ops._ptr_table(bufs)
        mp, wp = cuda_ops._ptr_table(masters), cuda_ops._ptr_table(my_w)
        shard = torch.empty(mine * per_mat, device=dev)
        shard_mats = [shard[i * per_mat: (i + 1) * per_mat].view(rows, cols) for i in range(mine)]
        sp = cuda_ops._ptr_table(shard_mats)
        gathered = torch.empty(numel, dtype=torch.bfloat16, device=dev)
        local_bf16 = torch.empty(mine * per_mat, dtype=torch.bfloat16, device=dev)
        lp = cuda_ops._ptr_table([local_bf16[i * per_mat: (i + 1) * per_mat].view(rows, cols) for i in range(mine)])
        iters = 20 if mb <= 64 else 6

        def rs_fused():
            barrier.sync()
            sumsq.zero_()
            c.rs_muon_prepare(gp, bp, packed, sumsq, rows, cols, cols, cols, 0.95, True, False, grads.deltas)

        def rs_fused_bf16():
            c.cast_bf16(grads.tensor[:numel], shadow.tensor[:numel])
            barrier.sync()
            sumsq.zero_()
            c.rs_muon_prepare(gp, bp, packed, sumsq, rows, cols, cols, cols, 0.95, True, False, shadow.deltas,
                              grad_base=grads.tensor, shadow=shadow.tensor)

        def rs_nccl():
            dist.reduce_scatter_tensor(shard, grads.tensor[:numel], op=dist.ReduceOp.AVG)
            sumsq.zero_()
            c.rs_muon_prepare(sp, bp, packed, sumsq, rows, cols, cols, cols, 0.95, True, False, [0])

        def ag_fused():
            c.muon_apply_push(mp, wp, packed, rows, cols, cols, cols, -0.01, False, weights.deltas)
            barrier.sync()

        def ag_nccl():
            c.muon_apply_push(mp, lp, packed, rows, cols, cols, cols, -0.01, False, [0])
            dist.all_gather_into_tensor(gathered, local_bf16)

        link_rs = numel * 4 / world * (world - 1)                    # bytes this GPU pulls from peers: its shard (1/world of the bucket) from every other rank
        link_ag = mine * per_mat * 2 * (world - 1)                   # bytes this GPU pushes: its shard to every other rank
        for name, fused, nccl, link in (("rs", rs_fused, rs_nccl, link_rs), ("ag", ag_fused, ag_nccl, link_ag)):
            if args.part not in (name, "all"):
                continue
            tf, tn = timed(fused, iters), timed(nccl, iters)
            hbm = mine * per_mat * ((4 * world + 4 + 4 + 2) if name == "rs" else (2 + 4 + 4 + 2 * world))
            roof_ms = max(link / (LINK_GBS * 1e6), hbm / 6552.6e6)
            results.append({"part": name, "bucket_mb": mb, "matrices": n_mats, "world": world, "fused_ms": tf, "nccl_ms": tn,
                            "speedup": tn / tf, "roofline_ms": roof_ms, "fraction_of_roofline": roof_ms / tf})
            if name == "rs" and world > 1:
                # bf16 on the wire (cast pass included): half the NVLink bytes, roofline likewise
                tb = timed(rs_fused_bf16, iters)
                roof_b = max(link / 2 / (LINK_GBS * 1e6), hbm / 6552.6e6)
                results[-1].update(fused_bf16_wire_ms=tb, speedup_bf16_wire=tn / tb, fraction_of_roofline_bf16_wire=roof_b / tb)
            if rank == 0:
                print(json.dumps(results[-1]), flush=True)
        del grads, weights, shadow


class _Shard:
    def __init__(self, world, experts, fused):
        self.ep_group, self.ep_size, self.num_experts, self.experts_per_rank = dist.group.WORLD, world, experts, experts // world
        self.ep_fused, self.ep_capacity_factor = fused, 0.0


def bench_ep(args, results):
    from gpt_moe_b200.parallel import ep_fused
    from gpt_moe_b200.parallel.ep import expert_parallel_moe
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    cases = [(16384, 768, 8, 1), (16384, 1024, 32, 2)] if args.quick else \
        [(t, d, e, k) for t in (4096, 16384, 65536) for d, e, k in ((768, 8, 1), (768, 32, 2), (1024, 64, 1), (1024, 32, 2))]
    for tokens, d, experts, top_k in cases:
        if experts % world:
            continue
        h = 3072 if experts == 8 else 1536 if experts == 32 else 1024
        n = experts // world
        torch.manual_seed(11 + rank)
        ups = [torch.randn(2 * h, d, device=dev).mul_(0.02).requires_grad_() for _ in range(n)]
        downs = [torch.randn(d, h, device=dev).mul_(0.02).requires_grad_() for _ in range(n)]
        hidden = torch.randn(tokens, d, device=dev).bfloat16().requires_grad_()
        # Zipf(1.1) popularity over experts, top-k distinct experts per token
        p = 1.0 / torch.arange(1, experts + 1, device=dev).float().pow(1.1)
        top_idx = torch.multinomial(p.expand(tokens, experts), top_k, replacement=False)
        gates = torch.full((tokens, top_k), 1.0 / top_k, device=dev).requires_grad_()
        g = torch.randn(tokens, d, device=dev).bfloat16()
        margs = dict(up_weights=ups, down_weights=downs, up_biases=None, down_biases=None, activation="swiglu",
                     up_precision=args.ep_precision, down_precision=args.ep_precision)

        shards = {True: _Shard(world, experts, True), False: _Shard(world, experts, False)}     # the fused path keys its receive buffer on the layer object

        def run(fused):
            out = expert_parallel_moe(shards[fused], hidden, top_idx, gates, margs)
            out.backward(g)
            for t in [hidden, gates] + ups + downs:
                t.grad = None

        iters = 10 if tokens <= 16384 else 4
        tf = timed(lambda: run(True), iters)
        tn = timed(lambda: run(False), iters)
        slots = tokens * top_k
        flops = 3 * 2 * slots * d * (3 * h)                                      # up (2h) + down (h), forward + two backward GEMMs each
        remote = slots * (world - 1) / world                                      # expected share of slots owned by another rank
        link = 4 * remote * d * 2                                                 # dispatch, combine, and both again in the backward
        roof_ms = max(flops / (GEMM_TFLOPS * 1e9), link / (LINK_GBS * 1e6))
        results.append({"part": "ep", "precision": args.ep_precision, "tokens_per_gpu": tokens, "d_model": d, "experts": experts, "top_k": top_k, "hidden": h, "world": world,
                        "fused_ms": tf, "nccl_ms": tn, "speedup": tn / tf, "roofline_ms": roof_ms, "fraction_of_roofline": roof_ms / tf})
        if rank == 0:
            print(json.dumps(results[-1]), flush=True)
        ep_fused.release_workspaces()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--part", default="all", choices=["rs", "ag", "ep", "all"])
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--ep-precision", default="default", choices=["default", "mxfp8"], help="precision of the expert projections in the ep part")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from gpt_moe_b200.ops import cuda_ops
    results = []
    if args.part in ("rs", "ag", "all"):
        bench_rs_ag(args, results)
    if args.part in ("ep", "all"):
        bench_ep(args, results)
    cuda_ops.check_status()
    if dist.get_rank() == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(results, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
