"""Expert-parallel dispatch / combine kernels on one GPU.

Two checks that need no second device: the whole fused function with a group of one (every row goes through the
"peer" stores and loads with a zero offset), and the kernels alone with two virtual ranks whose buffers are separate
allocations addressed through their pointer differences, phase by phase (no kernel waits on another, so running the
ranks one after the other is the same data flow as running them side by side).
"""
import pytest
import torch

from gpt_moe_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(scope="module")
def ops():
    from gpt_moe_b200.ops import cuda_ops
    cuda_ops.ext().reset_status()
    yield cuda_ops
    cuda_ops.check_status()


class _SoloMoE:
    ep_group, ep_size, ep_fused, ep_capacity_factor = None, 1, True, 1.0

    def __init__(self, experts):
        self.num_experts = self.experts_per_rank = experts


@pytest.mark.parametrize("top_k,experts,act", [(1, 8, "swiglu"), (2, 4, "relu2")])
def test_fused_ep_function_with_a_group_of_one(ops, top_k, experts, act):
    from gpt_moe_b200.parallel import ep_fused
    torch.manual_seed(5)
    m, d, h = 1000, 128, 256
    up_w = 2 * h if act == "swiglu" else h
    hidden = torch.randn(m, d, device="cuda").bfloat16().requires_grad_()
    logits = torch.randn(m, experts, device="cuda")
    logits[:, 1] = -1e4
    top_idx, gates, _ = ref.router_gates(logits, top_k, False)
    gates = gates.detach().requires_grad_()
    ups = [torch.randn(up_w, d, device="cuda").mul_(0.05).requires_grad_() for _ in range(experts)]
    downs = [torch.randn(d, h, device="cuda").mul_(0.05).requires_grad_() for _ in range(experts)]
    args = dict(up_weights=ups, down_weights=downs, up_biases=None, down_biases=None, activation=act)
    tensors = [hidden, gates] + ups + downs
    for _ in range(2):                                      # second pass reuses the buffers
        out = ep_fused.fused_expert_parallel_moe(_SoloMoE(experts), hidden, top_idx, gates, args)
        g = torch.randn_like(out)
        out.backward(g)
        got = [t.grad.clone() for t in tensors]
        for t in tensors:
            t.grad = None
        want = ops.moe_experts(hidden, top_idx, gates, ups, downs, None, None, act, "default", "default")
        want.backward(g)
        assert rel(out, want) < 1e-3
        for a, t in zip(got, tensors):
            assert rel(a, t.grad) < 1e-3
            t.grad = None
    ep_fused.release_workspaces()


def test_dispatch_and_combine_between_two_virtual_ranks(ops):
    c = ops.ext()
    torch.manual_seed(6)
    world, experts, per_rank, top_k, d, tokens = 2, 6, 3, 2, 64, 300
    cap = 2048 + per_rank * 256
    tables = [torch.zeros(world * experts, dtype=torch.int32, device="cuda") for _ in range(world)]
    recvs = [torch.full((cap, d), 7.0, device="cuda").bfloat16() for _ in range(world)]
    rets = [torch.empty(cap, d, device="cuda").bfloat16() for _ in range(world)]

    def deltas(bufs, me):
        return [b.data_ptr() - bufs[me].data_ptr() for b in bufs]

    hidden = [torch.randn(tokens, d, device="cuda").bfloat16() for _ in range(world)]
    idx, gates, routes = [], [], []
    for r in range(world):
        logits = torch.randn(tokens, experts, device="cuda")
        logits[:, 4] = -1e4                                   # expert 4 (rank 1) receives nothing
        ti, g, _ = ref.router_gates(logits, top_k, False)
        idx.append(ti.contiguous()); gates.append(g.float().contiguous())
        routes.append(c.route(idx[r], experts))
        c.ep_push_counts(routes[r][3], tables[r], deltas(tables, r), r)
    plans = [c.ep_plan(tables[r], world, r, experts, cap) for r in range(world)]
    assert torch.equal(tables[0], tables[1])
    route_rows = []
    for r in range(world):
        my_base, seg_ends, valid_ends, tiles, meta = plans[r]
        c.ep_zero_pads(recvs[r], seg_ends, valid_ends)
    for r in range(world):
        dest, _, local_seg_ends = routes[r][0], routes[r][1], routes[r][2]
        (rr,) = c.ep_dispatch(hidden[r], idx[r], dest, local_seg_ends, plans[r][0], None, None, recvs[r], deltas(recvs, r), per_rank)
        route_rows.append(rr)
    # every owner now holds, per local expert, the rows of rank 0 then rank 1 in token order, padded with zeros
    for owner in range(world):
        _, seg_ends, valid_ends, tiles, meta = plans[owner]
        start = 0
        for j in range(per_rank):
            e = owner * per_rank + j
            want = torch.cat([hidden[r][(idx[r] == e).any(dim=1).nonzero().flatten()] for r in range(world)])
            n = want.shape[0]
            assert valid_ends[j].item() == start + n
            assert torch.equal(recvs[owner][start:start + n], want)
            end = seg_ends[j].item()
            assert end == start + (n + 255) // 256 * 256
            assert recvs[owner][start + n:end].abs().max().item() == 0.0 if end > start + n else True
            assert (tiles[start // 128:end // 128] == j).all()
            start = end
        assert meta.tolist() == [start // 128, start]
    # "expert computation": y = 2 * x on the owner; combine pulls the rows back and applies the gates
    for r in range(world):
        rets[r].copy_(recvs[r].float().mul(2).bfloat16())
    for r in range(world):
        out, rows = c.ep_combine(rets[r], idx[r], route_rows[r], gates[r], True, deltas(rets, r), per_rank)
        want = 2 * hidden[r].float() * gates[r].sum(dim=1, keepdim=True)
        assert rel(out, want) < 4e-3
        assert torch.equal(rows.view(tokens, top_k, d)[:, 0], (2 * hidden[r].float()).bfloat16())
        # backward flavour of dispatch: rows scaled by the gate, gate gradient = <row, saved row>
        _, dg = c.ep_dispatch(hidden[r], idx[r], routes[r][0], routes[r][2], plans[r][0], gates[r], rows, recvs[r], deltas(recvs, r), per_rank)
        assert rel(dg, (hidden[r].float()[:, None, :] * rows.view(tokens, top_k, d).float()).sum(-1)) < 1e-3
    got = recvs[0][route_rows[0][0].item()] if idx[0][0, 0].item() < per_rank else recvs[1][route_rows[0][0].item()]
    assert rel(got, hidden[0][0].float() * gates[0][0, 0]) < 4e-3
