"""Worker of the multi-GPU engine test: run under `torch.distributed.run` with one process per GPU.

Trains a small GPT-MoE for a few steps with the fused peer-memory engine and with the NCCL engine on identical data
and prints one line `MULTI_GPU_ENGINE_OK` (rank 0) when losses and final weights agree.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run(fused: bool, steps: int = 4, ep: int = 1):
    from gpt_moe_b200.config import get_preset
    from gpt_moe_b200.runtime.trainer import Trainer
    from gpt_moe_b200.schedules.token import custom_schedule
    gc, tc = get_preset("small")
    gc.n_layers, gc.hidden_size, gc.attn_dim, gc.n_heads, gc.n_kv_heads = 2, 256, 256, 4, 4
    gc.mlp_hidden_dim, gc.num_experts, gc.weighted_main_path_init = 256, 4, 0.5
    tc.gpu_batch_size_train = tc.gpu_batch_size_val = 2
    tc.seq_len_train = tc.seq_len_val = 256
    tc.swa_values_schedule = {"fn": custom_schedule, "kwargs": {"values": [128]}}
    tc.kernel_warmup_train_steps = 0
    tc.use_fused_collectives = fused
    tc.overlap_grad_reduce = fused           # exercise the per-block flags and the second stream as well
    tc.expert_parallel_size = ep
    trainer = Trainer(gc, tc, device_type="cuda", quiet=True)
    want = "FusedEngine" if fused else "CudaHostEngine"
    assert type(trainer.engine).__name__ == want, type(trainer.engine).__name__
    gen = torch.Generator().manual_seed(100 + trainer.rank)
    losses = []
    for _ in range(steps):
        ids = torch.randint(0, gc.vocab_size, (2, 257), generator=gen)
        losses.append(trainer.train_step([(ids[:, :-1].contiguous(), ids[:, 1:].contiguous(), None)])["loss"])
    if hasattr(trainer.engine, "sync_masters"):
        trainer.engine.sync_masters()
    params = {n: p.detach().float().cpu().clone() for n, p in trainer.raw_gpt_model.named_parameters()}
    trainer.momentum = {k: v["momentum_buffer"].float() for k, v in trainer.engine.full_optimizer_state_dicts()["muon"]["state"].items()}
    return trainer, losses, params


class _Shard:
    """What `expert_parallel_moe` reads of a MoE layer."""

    def __init__(self, group, world, experts, fused):
        self.ep_group, self.ep_size, self.num_experts, self.experts_per_rank = group, world, experts, experts // world
        self.ep_fused, self.ep_capacity_factor = fused, float(world)


def check_expert_parallel_ops():
    """Fused dispatch/combine kernels and the NCCL all-to-all path against all experts computed locally."""
    import torch.distributed as dist
    from gpt_moe_b200.ops import cuda_ops, reference as ref
    from gpt_moe_b200.parallel.ep import expert_parallel_moe
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    experts, top_k, d, h, tokens = 4 * world, 2, 128, 256, 777
    torch.manual_seed(7)
    ups = [torch.randn(2 * h, d, device=dev).mul_(0.05).requires_grad_() for _ in range(experts)]
    downs = [torch.randn(d, h, device=dev).mul_(0.05).requires_grad_() for _ in range(experts)]
    torch.manual_seed(100 + rank)
    hidden = torch.randn(tokens, d, device=dev).bfloat16().requires_grad_()
    logits = torch.randn(tokens, experts, device=dev)
    logits[:, 1] = -1e4
    top_idx, gates, _ = ref.router_gates(logits, top_k, False)
    gates = gates.detach().requires_grad_()
    g = torch.randn(tokens, d, device=dev).bfloat16()
    tensors = [hidden, gates] + ups + downs

    def grads_of(out):
        out.backward(g)
        got = [t.grad.clone() if t.grad is not None else torch.zeros_like(t) for t in tensors]
        for t in tensors:
            t.grad = None
        return got

    want_out = cuda_ops.moe_experts(hidden, top_idx, gates, ups, downs, None, None, "swiglu", "default", "default")
    want = grads_of(want_out)
    for t in want[2:]:
        dist.all_reduce(t)                                    # an expert's gradient sums over the tokens of every rank
    lo, n = rank * (experts // world), experts // world
    args = dict(up_weights=ups[lo:lo + n], down_weights=downs[lo:lo + n], up_biases=None, down_biases=None, activation="swiglu",
                up_precision="default", down_precision="default")
    worst = 0.0
    for fused in (True, False, True):
        out = expert_parallel_moe(_Shard(dist.group.WORLD, world, experts, fused), hidden, top_idx, gates, args)
        got = grads_of(out)
        errs = [((out.float() - want_out.float()).norm() / want_out.float().norm()).item()]
        local = [0, 1] + [2 + lo + i for i in range(n)] + [2 + experts + lo + i for i in range(n)]
        for i in local:
            errs.append(((got[i].float() - want[i].float()).norm() / (want[i].float().norm() + 1e-6)).item())
        worst = max(worst, max(errs))
    # the same exchange with MXFP8 expert projections: against all experts computed locally with MXFP8 projections
    want_out = cuda_ops.moe_experts(hidden, top_idx, gates, ups, downs, None, None, "swiglu", "mxfp8", "mxfp8")
    want = grads_of(want_out)
    for t in want[2:]:
        dist.all_reduce(t)
    args_mx = dict(args, up_precision="mxfp8", down_precision="mxfp8")
    out = expert_parallel_moe(_Shard(dist.group.WORLD, world, experts, True), hidden, top_idx, gates, args_mx)
    got = grads_of(out)
    errs = [((out.float() - want_out.float()).norm() / want_out.float().norm()).item()]
    for i in [0, 1] + [2 + lo + i for i in range(n)] + [2 + experts + lo + i for i in range(n)]:
        errs.append(((got[i].float() - want[i].float()).norm() / (want[i].float().norm() + 1e-6)).item())
    worst = max(worst, max(errs))
    cuda_ops.check_status()
    return worst


def main():
    # One step from identical weights: the momentum buffers then hold the reduced gradients themselves.  Both engines ran the
    # same kernels on the same data, so they may differ only by the summation order of the cross-rank reduction.
    one_fused, _, _ = run(True, steps=1)
    one_nccl, _, _ = run(False, steps=1)
    from gpt_moe_b200.checkpointing.checkpoint import _optimizer_layout
    names = [n for group in _optimizer_layout(one_nccl.raw_gpt_model, one_nccl.optimizers["muon"])[1] for n in group]
    per_key = sorted(((one_fused.momentum[k] - one_nccl.momentum[k]).norm().item() / (one_nccl.momentum[k].norm().item() + 1e-12),
                      names[k], one_fused.momentum[k].norm().item(), one_nccl.momentum[k].norm().item()) for k in one_nccl.momentum)
    grad_err = per_key[-1][0]
    if one_nccl.rank == 0:
        print("reduced gradients, three worst (relative difference, name, |fused|, |nccl|):", per_key[-3:])
    grads_ok = set(one_fused.momentum) == set(one_nccl.momentum) and grad_err < 1e-4
    trainer, fused_losses, fused_params = run(True)
    _, nccl_losses, nccl_params = run(False)
    ep_err = check_expert_parallel_ops()
    _, ep_fused_losses, _ = run(True, ep=2)
    _, ep_nccl_losses, _ = run(False, ep=2)
    ep_ok = ep_err < 2e-2 and all(abs(a - b) < 3e-2 for a, b in zip(ep_fused_losses, ep_nccl_losses))
    ok = all(abs(a - b) < 3e-2 for a, b in zip(fused_losses, nccl_losses))
    worst = ("", 0.0)
    for n in fused_params:
        err = (fused_params[n] - nccl_params[n]).norm().item() / (nccl_params[n].norm().item() + 1e-3)
        if err > worst[1]:
            worst = (n, err)
    # both engines run the same kernels on the same reduced gradients; what differs is the summation order of the reduction
    # (and bf16 Polar Express amplifies that for the small router matrices): a few parts in a thousand after four steps
    worst_router = max([(n, (fused_params[n] - nccl_params[n]).norm().item() / (nccl_params[n].norm().item() + 1e-3))
                        for n in fused_params if "router" in n], key=lambda kv: kv[1], default=("", 0.0))
    worst_other = max([(n, (fused_params[n] - nccl_params[n]).norm().item() / (nccl_params[n].norm().item() + 1e-3))
                       for n in fused_params if "router" not in n], key=lambda kv: kv[1], default=("", 0.0))
    # After several Muon steps the weights are a poor yardstick: orthogonalisation lifts every singular value of the update to
    # about one, the noise directions of a small batch included, so summation-order differences of 1e-6 in the reduced gradient
    # come back as percents of the update (most of all in the 4 x 256 routers).  The tight check is the one on the reduced
    # gradients above; here only gross divergence is excluded.
    ok = ok and grads_ok and worst_other[1] < 5e-2 and worst_router[1] < 1.5e-1 and ep_ok
    flag = torch.tensor([1.0 if ok else 0.0], device=trainer.device)
    torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
    if trainer.rank == 0:
        print("fused losses", fused_losses)
        print("nccl  losses", nccl_losses)
        print("reduced gradients after one step: worst relative difference", grad_err)
        print("worst parameter difference (router)", worst_router, "(other)", worst_other)
        print("expert-parallel ops: worst relative error", ep_err)
        print("expert-parallel fused losses", ep_fused_losses)
        print("expert-parallel nccl  losses", ep_nccl_losses)
        print("MULTI_GPU_ENGINE_OK" if flag.item() == 1.0 else "MULTI_GPU_ENGINE_MISMATCH", flush=True)
    trainer.close()


if __name__ == "__main__":
    main()
