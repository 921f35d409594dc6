"""GPU kernels against the plain-PyTorch fp32 definitions in `ops.reference`.

Tolerances follow the reference's check scripts (`experiments/check_grouped.py:73-82`): relative L2 of
6e-3 for bf16 results, 1e-5 for fp32 statistics.
"""
import pytest
import torch

from gpt_moe_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
BF16_TOL = 6e-3


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(scope="module")
def ops():
    from gpt_moe_b200.ops import cuda_ops
    cuda_ops.ext().reset_status()
    yield cuda_ops
    cuda_ops.check_status()


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (1000, 776, 200), (4096, 2304, 768), (300, 8, 768), (64, 512, 128)])
def test_gemm_all_majors(ops, m, n, k):
    torch.manual_seed(0)
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    want = a.float() @ b.float().t()
    for a_mn in (False, True):
        for b_mn in (False, True):
            if (a_mn and m % 8) or (b_mn and n % 8):
                continue
            d = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
            ops.ext().gemm_bf16(a.t().contiguous() if a_mn else a, b.t().contiguous() if b_mn else b, d, a_mn, b_mn)
            assert rel(d, want) < BF16_TOL, (a_mn, b_mn)


def test_gemm_epilogue_batched_grouped(ops):
    torch.manual_seed(1)
    c = ops.ext()
    a = torch.randn(3, 256, 128, device="cuda").bfloat16()
    b = torch.randn(3, 512, 128, device="cuda").bfloat16()
    add = torch.randn(3, 256, 512, device="cuda").bfloat16()
    d = torch.empty(3, 256, 512, device="cuda", dtype=torch.bfloat16)
    c.gemm_bf16(a, b, d, False, False, 0.5, 2.0, add)
    assert rel(d, 0.5 * torch.bmm(a.float(), b.float().transpose(1, 2)) + 2.0 * add.float()) < BF16_TOL
    acc = torch.ones(256, 512, device="cuda")
    c.gemm_bf16(a[0], b[0], acc, False, False, 1.0, 0.0, None, True)
    assert rel(acc, 1 + a[0].float() @ b[0].float().t()) < 1e-5
    # ragged expert segments with an empty expert (segments padded to 256 rows, the unit of a CTA pair, by construction)
    counts, e, n, k = [0, 256, 768, 512], 4, 512, 256
    rows = sum(counts)
    x = torch.randn(rows, k, device="cuda").bfloat16()
    w = torch.randn(e, n, k, device="cuda").bfloat16()
    tiles = torch.tensor(sum([[i] * (cnt // 128) for i, cnt in enumerate(counts)], []), dtype=torch.int32, device="cuda")
    meta = torch.tensor([rows // 128, rows], dtype=torch.int32, device="cuda")
    y = torch.zeros(rows, n, device="cuda", dtype=torch.bfloat16)
    c.gemm_bf16(x, w, y, False, False, 1.0, 0.0, None, False, 1, tiles, meta, None)
    starts = [0, 0, 256, 1024]
    want = torch.cat([x[s:s + cnt].float() @ w[i].float().t() for i, (s, cnt) in enumerate(zip(starts, counts))])
    assert rel(y, want) < BF16_TOL
    dy = torch.randn(rows, n, device="cuda").bfloat16()
    ends = torch.tensor([0, 256, 1024, 1536], dtype=torch.int32, device="cuda")
    dw = torch.full((e, n, k), 7.0, device="cuda")
    c.gemm_bf16(dy, x, dw, True, True, 1.0, 0.0, None, False, 2, None, None, ends)
    want = torch.stack([dy[s:s + cnt].float().t() @ x[s:s + cnt].float() for s, cnt in zip(starts, counts)])
    assert rel(dw, want) < 1e-5
    assert dw[0].abs().max().item() == 0.0       # empty expert: exact zeros


def test_gemm_split_k_weight_gradient(ops):
    """Few output tiles and a long contraction: the K loop is shared by several CTAs and reduced by TMA."""
    torch.manual_seed(8)
    tokens, n, k = 8192, 256, 384
    dy = torch.randn(tokens, n, device="cuda").bfloat16()
    x = torch.randn(tokens, k, device="cuda").bfloat16()
    want = dy.float().t() @ x.float()
    dw = torch.full((n, k), 3.0, device="cuda")
    ops.ext().gemm_bf16(dy, x, dw, True, True)
    assert rel(dw, want) < 5e-5          # fp32 partial sums meet in arbitrary order
    ops.ext().gemm_bf16(dy, x, dw, True, True, 1.0, 0.0, None, True)
    assert rel(dw, 2 * want) < 5e-5


@pytest.mark.parametrize("d,dtype", [(768, torch.float32), (1024, torch.bfloat16), (128, torch.float32)])
def test_rmsnorm(ops, d, dtype):
    torch.manual_seed(2)
    x = torch.randn(4, 100, d, device="cuda").to(dtype).requires_grad_()
    w = (1 + 0.1 * torch.randn(d, device="cuda")).requires_grad_()
    y = ops.rms_norm(x, w, 1e-6)
    g = torch.randn_like(y)
    y.backward(g)
    x2, w2 = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    y2 = ref.rms_norm(x2, w2, 1e-6)
    y2.backward(g.float())
    assert rel(y, y2) < BF16_TOL and rel(x.grad, x2.grad) < BF16_TOL and rel(w.grad, w2.grad) < BF16_TOL


@pytest.mark.parametrize("d,rms", [(64, True), (32, False), (128, True)])
def test_rope_qknorm(ops, d, rms):
    torch.manual_seed(3)
    b, t, hq, hk = 2, 96, 4, 2
    q = torch.randn(b, t, hq, d, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(b, t, hk, d, device="cuda").bfloat16().requires_grad_()
    qs = torch.tensor([1.0, 0.5, 6.0, 2.0], device="cuda").view(1, hq, 1, 1).requires_grad_()   # 6.0 is clamped at 5
    ks = torch.tensor([1.5, 0.7], device="cuda").view(1, hk, 1, 1).requires_grad_()
    cos, sin = ref.rope_tables(d, 10000.0, t, device="cuda")
    oq, ok = ops.rope_qk_norm(q, k, cos, sin, qs, ks, 1e-6, rms, float("-inf"), 5.0)
    gq, gk = torch.randn_like(oq), torch.randn_like(ok)
    (oq.float() * gq.float()).sum().add((ok.float() * gk.float()).sum()).backward()
    q2, k2 = q.detach().float().requires_grad_(), k.detach().float().requires_grad_()
    qs2, ks2 = qs.detach().clone().requires_grad_(), ks.detach().clone().requires_grad_()
    rq, rk = ref.rope_qk_norm(q2, k2, cos, sin, qs2, ks2, 1e-6, rms, float("-inf"), 5.0)
    ((rq * gq.float()).sum() + (rk * gk.float()).sum()).backward()
    assert rel(oq, rq) < BF16_TOL and rel(ok, rk) < BF16_TOL
    assert rel(q.grad, q2.grad) < 1.5e-2 and rel(k.grad, k2.grad) < 1.5e-2
    assert rel(qs.grad, qs2.grad) < 1.5e-2 and rel(ks.grad, ks2.grad) < 1.5e-2
    assert qs.grad.view(-1)[2].item() == 0.0       # clamped scale receives no gradient


@pytest.mark.parametrize("top_k,experts,act", [(1, 8, "swiglu"), (2, 4, "relu2"), (2, 16, "swiglu")])
def test_moe_experts(ops, top_k, experts, act):
    torch.manual_seed(4)
    m, d, h = 1000, 128, 256
    up_w = 2 * h if act == "swiglu" else h
    hidden = torch.randn(m, d, device="cuda").bfloat16().requires_grad_()
    logits = torch.randn(m, experts, device="cuda")
    logits[:, 1] = -1e4                                   # expert 1 stays empty
    top_idx, gates, _ = ref.router_gates(logits, top_k, False)
    gates = gates.detach().requires_grad_()
    ups = [torch.randn(up_w, d, device="cuda").mul_(0.05).requires_grad_() for _ in range(experts)]
    downs = [torch.randn(d, h, device="cuda").mul_(0.05).requires_grad_() for _ in range(experts)]
    out = ops.moe_experts(hidden, top_idx, gates, ups, downs, None, None, act, "default", "default")
    g = torch.randn_like(out)
    out.backward(g)
    from gpt_moe_b200.ops import api
    hid2 = hidden.detach().float().cpu().requires_grad_()
    gates2 = gates.detach().cpu().requires_grad_()
    ups2 = [w.detach().bfloat16().float().cpu().requires_grad_() for w in ups]
    downs2 = [w.detach().bfloat16().float().cpu().requires_grad_() for w in downs]
    want = api.moe_experts(hid2, top_idx.cpu(), gates2, ups2, downs2, None, None, act, "default", "default")
    want.backward(g.float().cpu())
    assert rel(out.cpu(), want) < 1e-2
    assert rel(hidden.grad.cpu(), hid2.grad) < 2e-2 and rel(gates.grad.cpu(), gates2.grad) < 2e-2
    for a, b in zip(ups + downs, ups2 + downs2):
        assert rel(a.grad.cpu(), b.grad) < 2e-2
    assert ups[1].grad.abs().max().item() == 0.0          # empty expert: exact zero gradient


def test_linear_cross_entropy(ops):
    torch.manual_seed(5)
    rows, d, vocab = 300, 128, 50304
    x = torch.randn(rows, d, device="cuda").bfloat16().requires_grad_()
    w = torch.randn(vocab, d, device="cuda").mul_(0.02).requires_grad_()
    targets = torch.randint(0, vocab, (rows,), device="cuda")
    targets[::7] = -100
    loss = ops.linear_cross_entropy(x, w, targets, -100)
    loss.backward()
    x2 = x.detach().float().requires_grad_()
    w2 = w.detach().bfloat16().float().requires_grad_()
    want = ref.linear_cross_entropy(x2, w2, targets, -100)
    want.backward()
    assert abs(loss.item() - want.item()) < 2e-3
    assert rel(x.grad, x2.grad) < 2e-2 and rel(w.grad, w2.grad) < 2e-2


@pytest.mark.parametrize("m,k,batch", [(768, 768, 3), (768, 3072, 2), (640, 256, 2), (1024, 512, 1), (128, 256, 2), (264, 128, 1)])
def test_gemm_symmetric_mirror(ops, m, k, batch):
    """Triangle-and-mirror GEMMs of Polar Express: X X^T, and c A A + b A for a symmetric A, against fp32 matmuls."""
    torch.manual_seed(12)
    c = ops.ext()
    x = torch.randn(batch, m, k, device="cuda").bfloat16()
    a = torch.full((batch, m, m), float("nan"), device="cuda", dtype=torch.bfloat16)      # every element must be written
    c.gemm_bf16(x, x, a, symmetric=True)
    want = torch.bmm(x.float(), x.float().transpose(1, 2))
    assert rel(a, want) < BF16_TOL
    assert torch.equal(a, a.transpose(1, 2))
    full = torch.empty_like(a)
    c.gemm_bf16(x, x, full)
    assert torch.equal(torch.triu(a), torch.triu(full))          # the computed tiles are the ones the full product writes
    a.mul_(1.0 / k)
    b = torch.full_like(a, float("nan"))
    c.gemm_bf16(a, a, b, False, False, 0.7, -1.3, a, symmetric=True)
    want = 0.7 * torch.bmm(a.float(), a.float()) - 1.3 * a.float()
    assert rel(b, want) < BF16_TOL
    assert torch.equal(b, b.transpose(1, 2))


def test_polar_express_gemms(ops):
    """The tcgen05 Polar Express against the same iteration in torch bf16 (same rounding regime) and fp32."""
    torch.manual_seed(6)
    for shape in [(3, 256, 256), (2, 256, 1024), (1, 768, 3072)]:
        g = torch.randn(shape, device="cuda")
        x = (g / (g.norm(dim=(-2, -1), keepdim=True) * 1.02 + 1e-6)).bfloat16()
        got = ops.polar_express_bf16(x.clone())
        same_regime = ref.polar_express(g, dtype=torch.bfloat16)
        exact = ref.polar_express(g, dtype=torch.float32)
        assert rel(got, same_regime) < 5e-2, shape
        assert rel(got, exact) < 1.5e-1, shape
        sv = torch.linalg.svdvals(got.float())
        inside = ((sv > 0.5) & (sv < 1.3)).float().mean().item()      # the smallest few singular values converge last
        assert sv.max().item() < 1.3 and inside > 0.95, (shape, inside, sv.max().item())
        # the normalisation folded into the first iteration's epilogues: raw matrices plus their sums of squares
        raw = (g * 3e-4).bfloat16()
        sumsq = raw.float().pow(2).sum(dim=(-2, -1))
        folded = ops.polar_express_bf16(raw.clone(), sumsq)
        assert rel(folded, same_regime) < 5e-2, shape


@pytest.mark.parametrize("experts,top_k,full_softmax,dtype", [(8, 1, False, torch.bfloat16), (32, 2, False, torch.bfloat16),
                                                               (64, 1, False, torch.float32), (16, 4, True, torch.float32),
                                                               (100, 8, False, torch.float32)])
def test_router_kernel_matches_torch_router(ops, experts, top_k, full_softmax, dtype):
    """softmax + top-k + gates + load-balance loss in one kernel, and its backward, against the torch-op router."""
    torch.manual_seed(21)
    tokens = 1111
    # every row is a permutation of distinct values: the top-k choice has no ties in either precision
    base = torch.linspace(-3.0, 3.0, experts, device="cuda")
    order = torch.rand(tokens, experts, device="cuda").argsort(dim=1)
    logits = base[order].to(dtype).requires_grad_()
    top_idx, gates, balance = ops.router(logits, top_k, full_softmax, True, experts)
    want = logits.detach().clone().requires_grad_()
    w_idx, w_gates, w_probs = ref.router_gates(want, top_k, full_softmax)
    w_balance = ref.load_balance_loss(w_probs, w_idx, experts)
    assert torch.equal(top_idx, w_idx)
    assert torch.allclose(gates, w_gates, atol=1e-6, rtol=1e-5)
    assert torch.allclose(balance, w_balance, atol=1e-6, rtol=1e-5)
    dg = torch.randn_like(gates)
    (gates * dg).sum().add(balance * 0.37).backward()
    (w_gates * dg).sum().add(w_balance * 0.37).backward()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert rel(logits.grad, want.grad) < tol
    # no balance loss requested: nothing but the gates flows back
    logits.grad = None
    i2, g2, b2 = ops.router(logits, top_k, full_softmax, False, experts)
    assert b2 is None and torch.equal(i2, top_idx)


def test_polar_express_on_router_sized_matrices(ops):
    """Matrices far below one tile (a router: experts x hidden) run through the same batched tcgen05 iteration; the fused
    engine relies on it to keep routers off the host path."""
    torch.manual_seed(16)
    for shape in [(12, 8, 768), (5, 64, 1024), (3, 16, 256)]:
        g = torch.randn(shape, device="cuda")
        raw = (g * 1e-3).bfloat16()
        sumsq = raw.float().pow(2).sum(dim=(-2, -1))
        got = ops.polar_express_bf16(raw.clone(), sumsq)
        want = ref.polar_express(raw.float(), dtype=torch.float32)
        assert got.shape == raw.shape and torch.isfinite(got.float()).all()
        assert rel(got, want) < 1.5e-1, (shape, rel(got, want))


def test_adamw_sharded_tracks_torch_adamw_over_a_thousand_steps(ops):
    """The sharded AdamW kernel (IEEE division and square root, fp32 moments) against `torch.optim.AdamW` on the same
    gradient stream for 1000 steps: parameters stay within float rounding of each other."""
    c = ops.ext()
    torch.manual_seed(17)
    n = 4096
    p = torch.randn(n, device="cuda") * 0.02
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    grads = torch.zeros(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    decay = torch.full((n,), 0.1, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(18)
    for step in range(1, 1001):
        g = torch.randn(n, device="cuda", generator=gen) * (1.0 + 0.5 * torch.sin(torch.tensor(step / 50.0)).item())
        grads.copy_(g)
        ref_p.grad = g.clone()
        opt.step()
        c.adamw_sharded(p, grads, m, v, decay, 0, n, 3e-3, 0.9, 0.95, 1e-8, step, [0], [0])
    err = (p - ref_p.detach()).abs().max().item()
    assert err < 2e-5, err


def test_adamw_and_muon_steps(ops):
    from gpt_moe_b200.optim import AdamW, Muon
    torch.manual_seed(7)
    shapes = [(256, 256), (512, 256), (256, 1024), (8, 256), (768, 256)]
    ps = [torch.randn(s).mul_(0.02) for s in shapes]
    gs = [torch.randn(s) for s in shapes]
    gpu = [p.clone().cuda().requires_grad_() for p in ps]
    for p, g in zip(gpu, gs):
        p.grad = g.clone().cuda()
    opt = Muon(gpu, lr=0.02, momentum=0.95, nesterov=True, backend="polarexpress")
    opt.step()
    for p, p0, g in zip(gpu, ps, gs):
        # first step: buf = g, u = g + 0.95 g; the update is -lr*sqrt(max(shape)) * polar(u); (768,256) is split into 3 squares
        u = (g * 1.95).cuda()
        parts = u.split(u.shape[1]) if u.shape[0] == 3 * u.shape[1] else [u]
        want = torch.cat([ref.polar_express(q, dtype=torch.bfloat16).float() * (-0.02 * max(q.shape) ** 0.5) for q in parts])
        if min(p.shape) < 128:
            # a handful of singular values: two bf16 iterations with different rounding points scatter more than on a large matrix,
            # so the router-sized case is held against the fp32 iteration instead
            exact = ref.polar_express(u, dtype=torch.float32).float() * (-0.02 * max(u.shape) ** 0.5)
            assert rel(p.detach() - p0.cuda(), exact) < 1.5e-1, (tuple(p.shape), rel(p.detach() - p0.cuda(), exact))
        else:
            assert rel(p.detach() - p0.cuda(), want) < 6e-2, tuple(p.shape)
        assert rel(opt.state[p]["momentum_buffer"], g.cuda()) < 1e-6
    cpu = [p.clone().requires_grad_() for p in ps]
    gpu = [p.clone().cuda().requires_grad_() for p in ps]
    ac, ag = AdamW(cpu, lr=1e-2, weight_decay=0.1), AdamW(gpu, lr=1e-2, weight_decay=0.1)
    for _ in range(3):
        for c, g_, gr in zip(cpu, gpu, gs):
            c.grad, g_.grad = gr.clone(), gr.clone().cuda()
        ac.step(); ag.step()
    for c, g_, p0 in zip(cpu, gpu, ps):
        assert rel(g_.detach().cpu() - p0, c.detach() - p0) < 1e-4
    assert float(ag.state_dict()["state"][0]["step"]) == 3.0


@pytest.mark.parametrize("t,window,hq,hk", [(256, 1000, 2, 2), (512, 128, 4, 2), (1024, 300, 2, 1), (384, 0, 2, 2)])
def test_attention_forward_kernel(ops, t, window, hq, hk):
    torch.manual_seed(9)
    b, d = 2, 64
    packed = torch.randn(b, t, (hq + 2 * hk) * d, device="cuda").bfloat16()      # q | k | v columns of one projection output
    q = packed[..., : hq * d].unflatten(-1, (hq, d))
    k = packed[..., hq * d: (hq + hk) * d].unflatten(-1, (hk, d))
    v = packed[..., (hq + hk) * d:].unflatten(-1, (hk, d))
    out, lse = ops.ext().attn_fwd(q, k, v, window, d ** -0.5)
    want = ref.attention(q.float(), k.float(), v.float(), causal=True, window=window)
    assert rel(out, want) < 1e-2
    # log-sum-exp of the scaled, masked scores
    rep = hq // hk
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float().repeat_interleave(rep, dim=2)) * d ** -0.5
    keep = ref.attention_mask(t, "cuda", True, window)
    assert torch.allclose(lse, torch.logsumexp(s.masked_fill(~keep, float("-inf")), dim=-1), atol=2e-2)


@pytest.mark.parametrize("t,window,hq,hk,gain,softcap", [
    (256, 1000, 2, 2, 1.0, 0.0), (512, 128, 4, 2, 1.0, 0.0), (1024, 300, 2, 1, 1.0, 0.0), (2048, 1024, 2, 1, 1.0, 0.0), (512, 0, 2, 2, 1.0, 0.0),
    (768, 77, 2, 2, 1.0, 0.0), (2048, 5000, 1, 1, 1.0, 0.0), (1024, 500, 2, 2, 6.0, 0.0), (2048, 1024, 2, 2, 12.0, 0.0), (512, 200, 2, 1, 3.0, 20.0)])
def test_attention_forward_two_query_tiles_per_cta(ops, t, window, hq, hk, gain, softcap):
    """The forward kernel that shares key/value tiles between two query tiles and keeps O in TMEM: against the fp32 reference and
    against the single-tile kernel.  `gain` scales the queries so that row maxima keep growing from tile to tile (the row's
    reference maximum moves and O is rescaled in TMEM) or stay within the slack (a stale reference is used)."""
    torch.manual_seed(11)
    b, d = 2, 64
    packed = torch.randn(b, t, (hq + 2 * hk) * d, device="cuda")
    packed[..., : hq * d] *= gain
    packed = packed.bfloat16()
    q = packed[..., : hq * d].unflatten(-1, (hq, d))
    k = packed[..., hq * d: (hq + hk) * d].unflatten(-1, (hk, d))
    v = packed[..., (hq + hk) * d:].unflatten(-1, (hk, d))
    c = ops.ext()
    out, lse = c.attn_fwd(q, k, v, window, d ** -0.5, softcap)
    one, lse_one = c.attn_fwd(q, k, v, window, d ** -0.5, softcap, None, False, True)
    ops.check_status()
    want = ref.attention(q.float(), k.float(), v.float(), causal=True, window=window, softcap_value=softcap, tanh_backend="exact")
    assert rel(out, want) < 1e-2
    assert rel(out, one) < 6e-3
    assert torch.allclose(lse, lse_one, atol=2e-2, rtol=1e-3)
    if softcap == 0.0:
        rep = hq // hk
        s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float().repeat_interleave(rep, dim=2)) * d ** -0.5
        keep = ref.attention_mask(t, "cuda", True, window)
        assert torch.allclose(lse, torch.logsumexp(s.masked_fill(~keep, float("-inf")), dim=-1), atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("t,window,hq,hk", [(256, 1000, 2, 2), (512, 128, 4, 2), (1024, 300, 2, 1), (384, 0, 2, 2)])
def test_attention_backward_kernel(ops, t, window, hq, hk):
    from gpt_moe_b200.ops import attention_tc
    torch.manual_seed(10)
    b, d = 2, 64
    packed = torch.randn(b, t, (hq + 2 * hk) * d, device="cuda").bfloat16().requires_grad_()
    q, k, v = ops.split_qkv(packed, hq, hk, d)
    assert attention_tc.supported(q, k, v, 0.0)
    out = attention_tc.attention(q, k, v, window=window, scale=None)
    g = torch.randn_like(out)
    out.backward(g)
    ref_in = packed.detach().float().requires_grad_()
    rq = ref_in[..., : hq * d].unflatten(-1, (hq, d))
    rk = ref_in[..., hq * d: (hq + hk) * d].unflatten(-1, (hk, d))
    rv = ref_in[..., (hq + hk) * d:].unflatten(-1, (hk, d))
    want = ref.attention(rq, rk, rv, causal=True, window=window)
    want.backward(g.float())
    assert rel(out, want) < 1e-2
    got, exp = packed.grad.float(), ref_in.grad
    for name, sl in (("dq", slice(0, hq * d)), ("dk", slice(hq * d, (hq + hk) * d)), ("dv", slice((hq + hk) * d, None))):
        if exp[..., sl].norm().item() < 1e-6:          # window 0: a single visible key makes dq and dk vanish exactly
            assert got[..., sl].abs().max().item() < 1e-4, name
        else:
            assert rel(got[..., sl], exp[..., sl]) < 2e-2, name


@pytest.mark.parametrize("t,window,hq,hk,softcap,docs", [(256, 1000, 2, 2, 0.0, False), (512, 128, 4, 2, 0.0, False), (1024, 300, 2, 1, 0.0, False),
                                                         (2048, 1024, 4, 2, 0.0, False), (384, 0, 2, 2, 0.0, False), (640, 77, 2, 1, 0.0, False),
                                                         (1024, 400, 2, 2, 15.0, False), (1024, 5000, 2, 1, 0.0, True)])
def test_attention_backward_pipelined_matches_unpipelined(ops, t, window, hq, hk, softcap, docs):
    """The backward kernel that issues the next tile's score products ahead of the current gradient products forms the same
    P and dS as the kernel that issues everything in program order; only the order of the fp32 additions into dQ differs."""
    from gpt_moe_b200.ops import attention_tc
    torch.manual_seed(12)
    b, d = 2, 64
    c = ops.ext()
    packed = torch.randn(b, t, (hq + 2 * hk) * d, device="cuda").bfloat16()
    q, k, v = ops.split_qkv(packed, hq, hk, d)
    doc_start = None
    if docs:
        ids = torch.cumsum((torch.rand(b, t, device="cuda") < 0.01).long(), dim=1)
        doc_start = attention_tc.document_starts(ids)
    out, lse = c.attn_fwd(q, k, v, min(window, t), d ** -0.5, softcap, doc_start)
    g = torch.randn_like(out)
    results = []
    for unpipelined in (False, True):
        dk = torch.empty(b, t, hk, d, device="cuda", dtype=torch.bfloat16)
        dv = torch.empty(b, t, hk, d, device="cuda", dtype=torch.bfloat16)
        dq = c.attn_bwd(q, k, v, out, g, lse, dk, dv, min(window, t), d ** -0.5, softcap, doc_start, unpipelined)
        ops.check_status()
        results.append((dq, dk.float(), dv.float()))
    for got, want, name in zip(results[0], results[1], ("dq", "dk", "dv")):
        scale = want.abs().max().item()
        assert (got - want).abs().max().item() <= 2e-2 * scale + 1e-6, name
        if scale > 1e-6:
            assert rel(got, want) < 2e-3, name


@pytest.mark.parametrize("t,window,hq,hk", [(256, 1000, 2, 2), (512, 128, 4, 2), (1024, 2000, 2, 1)])
def test_attention_kernels_wide_query_key_heads(ops, t, window, hq, hk):
    """Multi-head latent attention shape: 128-wide query / key heads (content + rotary), 64-wide value heads."""
    from gpt_moe_b200.ops import attention_tc
    torch.manual_seed(11)
    b, dqk, dv = 2, 128, 64
    q = torch.randn(b, t, hq, dqk, device="cuda").mul_(0.5).bfloat16().requires_grad_()
    k = torch.randn(b, t, hk, dqk, device="cuda").mul_(0.5).bfloat16().requires_grad_()
    v = torch.randn(b, t, hk, dv, device="cuda").bfloat16().requires_grad_()
    assert attention_tc.supported(q, k, v, 0.0)
    out = attention_tc.attention(q, k, v, window=window, scale=None)
    g = torch.randn_like(out)
    out.backward(g)
    rq, rk, rv = (x.detach().float().requires_grad_() for x in (q, k, v))
    want = ref.attention(rq, rk, rv, causal=True, window=window)
    want.backward(g.float())
    assert out.shape == (b, t, hq, dv)
    assert rel(out, want) < 1e-2
    for name, got, exp in (("dq", q.grad, rq.grad), ("dk", k.grad, rk.grad), ("dv", v.grad, rv.grad)):
        assert rel(got, exp) < 2e-2, name


def test_kernels_are_bitwise_deterministic(ops):
    """No atomics decide a result: the same launch twice gives the same bits (GEMM, grouped GEMM, routing, norms, CE)."""
    torch.manual_seed(12)
    c = ops.ext()
    a = torch.randn(1000, 768, device="cuda").bfloat16(); b = torch.randn(776, 768, device="cuda").bfloat16()
    outs = []
    for _ in range(2):
        d = torch.empty(1000, 776, device="cuda", dtype=torch.bfloat16)
        c.gemm_bf16(a, b, d)
        idx = torch.randint(0, 8, (4096, 2), device="cuda", generator=torch.Generator("cuda").manual_seed(5))
        route = c.route(idx, 8)
        x = torch.randn(4096, 768, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
        dy = torch.randn(4096, 768, device="cuda", generator=torch.Generator("cuda").manual_seed(2)).bfloat16()
        w = torch.ones(768, device="cuda")
        y, rstd, _ = c.rmsnorm_fwd(x, w, 1e-6)
        dx, dwn = c.rmsnorm_bwd(dy, x, w, rstd, None)
        logits = torch.randn(512, 50304, device="cuda", generator=torch.Generator("cuda").manual_seed(3)).bfloat16()
        tg = torch.randint(0, 50304, (512,), device="cuda", generator=torch.Generator("cuda").manual_seed(4))
        loss = c.ce_fwd_bwd(logits, tg, torch.ones(1, device="cuda"), -100, True)
        used = int(route[5][1].item())                                      # rows beyond the padded segments are never written
        outs.append([d, route[0], route[1][:used], route[2], route[4][: used // 128], y, dx, dwn, logits] + [t for t in (loss if isinstance(loss, (list, tuple)) else [loss])])
    for first, second in zip(*outs):
        assert torch.equal(first, second)


def test_bounded_wait_gives_up_and_reports(ops):
    """A wait on a flag that nothing sets runs out of its budget (about a second), records its code in the status word
    and returns: the context stays usable and the host sees the failure."""
    c = ops.ext()
    c.reset_status()
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    c.flag_signal(flags, [0], 1, 7)                       # slot 1 is published, slot 0 never is
    c.flag_wait(flags, 1, 1, 7)                           # satisfied at once
    torch.cuda.synchronize()
    assert c.read_status() == 0 and flags.tolist() == [0, 7, 0, 0]
    c.flag_wait(flags, 0, 1, 7)                           # nobody writes flags[0]
    torch.cuda.synchronize()
    assert c.read_status() == 601
    with pytest.raises(RuntimeError):
        ops.check_status()
    assert c.read_status() == 0                           # check_status clears the word
    a = torch.randn(128, 64, device="cuda").bfloat16()
    d = torch.empty(128, 128, device="cuda", dtype=torch.bfloat16)
    c.gemm_bf16(a, a, d)                                  # kernels still run afterwards
    assert rel(d, a.float() @ a.float().t()) < BF16_TOL


def test_peer_barrier_completes_alone_and_gives_up_on_a_missing_peer(ops):
    """The device-side barrier on one GPU: a group of one passes at once and bumps its epoch; a group of two whose second
    member's slot nothing writes runs out of its (shortened) budget, records 601 and returns with the context usable.  Flag
    values can also come from a device word."""
    c = ops.ext()
    c.reset_status()
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    c.peer_barrier(flags, [0], 0, epoch)
    c.peer_barrier(flags, [0], 0, epoch)
    torch.cuda.synchronize()
    assert c.read_status() == 0 and epoch.item() == 2 and flags.tolist() == [2, 0, 0, 0]
    c.peer_barrier(flags, [0, 0], 0, epoch, 200_000_000)      # "rank 1" shares this table and never publishes into slot 1
    torch.cuda.synchronize()
    assert c.read_status() == 601 and flags.tolist() == [3, 0, 0, 0]
    c.reset_status()
    word = torch.zeros(1, dtype=torch.int32, device="cuda")
    c.bump_word(word)
    c.bump_word(word)
    c.flag_signal(flags, [0], 2, 0, word)                     # value read from the device word
    c.flag_wait(flags, 2, 1, 0, word)
    torch.cuda.synchronize()
    assert c.read_status() == 0 and flags.tolist() == [3, 0, 2, 0]


@pytest.mark.parametrize("dqk,window", [(64, 200), (128, 2000)])
def test_attention_kernels_with_logit_softcapping(ops, dqk, window):
    """softcap * tanh(scale * s / softcap) before the softmax, forward and backward (hardware tanh.approx)."""
    from gpt_moe_b200.ops import attention_tc
    torch.manual_seed(13)
    b, t, hq, hk, cap = 2, 512, 4, 2, 15.0
    q = torch.randn(b, t, hq, dqk, device="cuda").mul_(2.0).bfloat16().requires_grad_()      # large logits so the cap matters
    k = torch.randn(b, t, hk, dqk, device="cuda").mul_(2.0).bfloat16().requires_grad_()
    v = torch.randn(b, t, hk, 64, device="cuda").bfloat16().requires_grad_()
    assert attention_tc.supported(q, k, v, cap)
    out = attention_tc.attention(q, k, v, window=window, scale=None, softcap=cap)
    g = torch.randn_like(out)
    out.backward(g)
    rq, rk, rv = (x.detach().float().requires_grad_() for x in (q, k, v))
    want = ref.attention(rq, rk, rv, causal=True, window=window, softcap_value=cap, tanh_backend="exact")
    want.backward(g.float())
    plain = ref.attention(rq.detach(), rk.detach(), rv.detach(), causal=True, window=window)
    assert rel(plain, want) > 5e-2                        # the cap changes the result on this input
    assert rel(out, want) < 1.5e-2
    for name, got, exp in (("dq", q.grad, rq.grad), ("dk", k.grad, rk.grad), ("dv", v.grad, rv.grad)):
        assert rel(got, exp) < 3e-2, name


@pytest.mark.parametrize("dqk,window", [(64, 300), (64, 5000), (128, 5000)])
def test_attention_kernels_with_document_masking(ops, dqk, window):
    """Queries see only keys of their own document (documents = contiguous runs), combined with the causal window."""
    from gpt_moe_b200.ops import attention_tc
    torch.manual_seed(14)
    b, t, hq, hk = 2, 640, 2, 1
    q = torch.randn(b, t, hq, dqk, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(b, t, hk, dqk, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(b, t, hk, 64, device="cuda").bfloat16().requires_grad_()
    ends = torch.zeros(b, t, dtype=torch.long, device="cuda")
    for row, cuts in enumerate(([5, 130, 131, 400], [127, 128, 500, 639])):      # documents of very different lengths, cuts at tile edges too
        ends[row, cuts] = 1
    docs = ends.cumsum(dim=1) - ends                                               # the end-of-sequence token belongs to its document
    assert attention_tc.document_starts(docs)[0, 131].item() == 131 and attention_tc.document_starts(docs)[0, 399].item() == 132
    out = attention_tc.attention(q, k, v, window=window, scale=None, document_ids=docs)
    g = torch.randn_like(out)
    out.backward(g)
    rq, rk, rv = (x.detach().float().requires_grad_() for x in (q, k, v))
    want = ref.attention(rq, rk, rv, causal=True, window=window, document_ids=docs)
    want.backward(g.float())
    assert rel(out, want) < 1e-2
    for name, got, exp in (("dq", q.grad, rq.grad), ("dk", k.grad, rk.grad), ("dv", v.grad, rv.grad)):
        assert rel(got, exp) < 2e-2, name


@pytest.mark.parametrize("t,hkv,r,dr,window,softcap", [(1, 16, 512, 64, None, 0.0), (3, 4, 512, 64, 100, 0.0), (2, 16, 256, 16, None, 30.0),
                                                       (1, 8, 768, 16, 37, 0.0)])
def test_mla_decode_kernel_matches_torch_decode(ops, t, hkv, r, dr, window, softcap):
    """Split-K latent-cache decode + log-sum-exp merge against the torch formulation of the same absorbed-weight attention."""
    from gpt_moe_b200.models.mla import api_mla_decode
    torch.manual_seed(31)
    b, h, s_len, start = 2, 16, 333, 333 - t
    q_latent = torch.randn(b, t, h, r, device="cuda") * 0.2
    q_rope = torch.randn(b, t, h, dr, device="cuda") * 0.2
    cache = torch.randn(b, 400, r, device="cuda").bfloat16()                 # the views below are shorter than the cache
    rope = torch.randn(b, 400, dr, device="cuda").bfloat16()
    gain = (torch.rand(b, 400, hkv, device="cuda") + 0.5).bfloat16()
    args = (start, 0.11, softcap, "exact", window)
    got = api_mla_decode(q_latent, q_rope, cache[:, :s_len], rope[:, :s_len], gain[:, :s_len], *args)
    want = api_mla_decode(q_latent, q_rope, cache[:, :s_len].float(), rope[:, :s_len].float(), gain[:, :s_len].float(), *args)
    assert ops.path_counts().get("mla_decode:kernel", 0) >= 1
    assert got.shape == want.shape and rel(got, want) < 2e-3, rel(got, want)


def test_bounds_checked_build_skips_bad_indices(ops):
    """Only in the bounds-checked build (GM_CHECK_BOUNDS=1 selects `_C_checked.so`): an expert id, a routed row or a target class
    outside its range is not used as an address; the kernel skips the access, records a code, and the context stays usable."""
    c = ops.ext()
    if not c.bounds_checked():
        pytest.skip("normal build: indices are not checked (run with GM_CHECK_BOUNDS=1)")
    assert c.read_bounds_status() == 0
    idx = torch.randint(0, 4, (512, 1), device="cuda")
    idx[7, 0] = 9                                            # four experts: 9 does not exist
    c.route(idx, 4)
    torch.cuda.synchronize()
    assert c.read_bounds_status() == 901
    assert c.read_bounds_status() == 0                       # reading clears the word
    logits = torch.randn(64, 512, device="cuda").bfloat16()
    targets = torch.randint(0, 512, (64,), device="cuda")
    targets[3] = 512                                         # one past the last class: treated as an ignored row
    loss = c.ce_fwd_bwd(logits, targets, torch.ones(1, device="cuda"), -100, True)
    torch.cuda.synchronize()
    assert c.read_bounds_status() == 905 and torch.isfinite(loss).all() and loss[3].item() == 0.0
    a = torch.randn(128, 64, device="cuda").bfloat16()
    d = torch.empty(128, 128, device="cuda", dtype=torch.bfloat16)
    c.gemm_bf16(a, a, d)                                     # kernels still run afterwards
    assert rel(d, a.float() @ a.float().t()) < BF16_TOL


@pytest.mark.parametrize("precision", ["default", "mxfp8"])
def test_linear_accepts_non_contiguous_inputs_and_selective_backward(ops, precision):
    """Cases of the reference's check scripts: a strided view as input (every other row of a wider tensor), a gradient requested
    for the weights only / the input only, and fp32 as well as bf16 activations."""
    torch.manual_seed(41)
    big = torch.randn(2 * 192, 2 * 256, device="cuda")
    w1 = (torch.randn(256, 256, device="cuda") * 0.05).requires_grad_()
    w2 = (torch.randn(128, 256, device="cuda") * 0.05).requires_grad_()
    tol = 4e-2 if precision == "mxfp8" else BF16_TOL
    for dtype in (torch.float32, torch.bfloat16):
        view = big.to(dtype)[::2, ::2]                          # non-contiguous in both dimensions
        assert not view.is_contiguous()
        x = view.detach().requires_grad_()
        y = ops.linear_multi(x, (w1, w2), precision)
        want = x.detach().float().bfloat16().float() @ torch.cat((w1, w2)).detach().bfloat16().float().t()
        assert rel(y, want) < tol
        # only the weights need a gradient
        x_nograd = view.detach()
        y2 = ops.linear_multi(x_nograd, (w1, w2), precision)
        g = torch.randn_like(y2)
        y2.backward(g)
        dw = g.float().t() @ x_nograd.float().bfloat16().float()
        assert rel(torch.cat((w1.grad, w2.grad)), dw) < 2e-2
        w1.grad = w2.grad = None
        # only the input needs a gradient
        w1f, w2f = w1.detach(), w2.detach()
        y3 = ops.linear_multi(x, (w1f, w2f), precision)
        y3.backward(g)
        dx = g.float() @ torch.cat((w1f, w2f)).bfloat16().float()
        assert rel(x.grad, dx) < tol
        x.grad = None


def test_rope_qknorm_backward_with_only_the_queries_used(ops):
    """Selective-output backward: the loss touches the rotated queries only; keys get zero gradient, the packed gradient that
    reaches the projection is complete, and the key scale's gradient is exactly zero."""
    torch.manual_seed(42)
    t, hq, hk, d = 256, 4, 2, 64
    qkv = torch.randn(t, (hq + 2 * hk) * d, device="cuda").bfloat16().requires_grad_()
    pos = torch.arange(128, device="cuda").float()[:, None] * (10000.0 ** (-torch.arange(d // 2, device="cuda").float() / (d // 2)))[None, :]
    cos, sin = pos.cos().contiguous(), pos.sin().contiguous()
    qs = torch.full((1, hq, 1, 1), 1.2, device="cuda", requires_grad=True)
    ks = torch.full((1, hk, 1, 1), 0.8, device="cuda", requires_grad=True)
    out = ops.rope_qk_norm_packed(qkv, cos, sin, qs, ks, 128, hq, hk, d, 1e-6, True, -1e9, 5.0)
    q, k, v = ops.split_qkv(out.view(2, 128, -1), hq, hk, d)
    q.float().square().sum().backward()
    grad = qkv.grad.view(t, hq + 2 * hk, d)
    assert grad[:, :hq].abs().max().item() > 0
    assert grad[:, hq:].abs().max().item() == 0.0
    assert qs.grad is not None and ks.grad.abs().max().item() == 0.0


def test_quantised_weights_are_cached_across_micro_steps_and_refreshed_after_an_update(ops):
    """The reference's cached-weight case: four accumulation micro-steps reuse one quantisation of the weights, an optimizer
    update (announced through `mark_parameters_updated`) makes the next use quantise again."""
    from gpt_moe_b200.ops import mxfp8
    torch.manual_seed(43)
    w = (torch.randn(256, 256, device="cuda") * 0.05).requires_grad_()
    x = torch.randn(128, 256, device="cuda").bfloat16()
    mxfp8.clear_quantized_weights()
    first = mxfp8._quantized_weight((w,), stack=False)
    for _ in range(4):
        ops.linear_multi(x, (w,), "mxfp8").float().sum().backward()
        assert mxfp8._quantized_weight((w,), stack=False)[1] is first[1]             # same cached tensor object
    with torch.no_grad():
        w.mul_(0.5)
    ops.mark_parameters_updated()
    second = mxfp8._quantized_weight((w,), stack=False)
    assert second[1] is not first[1]
    want_q, _ = ref.mxfp8_quantize(w.detach().bfloat16().float(), -1)
    assert torch.equal(second[1].view(torch.float8_e4m3fn).float(), want_q.float())


def test_mma_issue_bench_reports_device_clocks(ops):
    """The issue-rate probe runs, completes (bounded wait) and shows the instruction time growing with N only above the floor."""
    c = ops.ext()
    issue256, done256 = c.mma_issue_bench(1, 64)       # M128 N256
    issue64, done64 = c.mma_issue_bench(2, 64)         # M128 N64
    ops.check_status()
    assert 0 < issue256 <= done256 and 0 < issue64 <= done64
    assert done64 < done256 < 8 * done64


def test_output_guards_report_a_write_past_an_output(ops):
    """Bounds-checked build with GM_CANARIES=1: the bindings' allocations carry 256 guard bytes on either side.  A byte past the
    payload is changed here from the host side (a torch write into the underlying storage, standing in for a kernel that stored
    one element too far) and the status check reports it; a clean call afterwards reports nothing."""
    c = ops.ext()
    if not (c.bounds_checked() and c.output_guards_enabled()):
        pytest.skip("guard bytes exist only in the bounds-checked build with GM_CANARIES=1")
    ops.check_status()                                     # forget what earlier tests allocated
    x = torch.randn(256, 128, device="cuda").bfloat16()
    q, sf = c.mxfp8_quantize(x)
    assert q.storage_offset() == 256
    raw = torch.empty(0, dtype=torch.uint8, device="cuda").set_(q.untyped_storage())
    assert int(raw[255]) == 0xA5 and int(raw[256 + q.numel()]) == 0xA5
    raw[256 + q.numel()] = 0
    with pytest.raises(RuntimeError, match="guard bytes"):
        ops.check_status()
    q2, _ = c.mxfp8_quantize(x)
    ops.check_status()
    assert torch.equal(q, q2)


def test_attention_reads_a_device_resident_window(ops):
    """The look-back may live in a one-element int32 tensor that the kernels read on the device: the same call then follows a
    window schedule (a `fill_`) without a new host argument.  Forward and backward, both kernels of each direction."""
    torch.manual_seed(13)
    b, t, h, d = 2, 1024, 2, 64
    c = ops.ext()
    packed = torch.randn(b, t, 3 * h * d, device="cuda").bfloat16()
    q, k, v = ops.split_qkv(packed, h, h, d)
    word = torch.zeros((), dtype=torch.int32, device="cuda")
    for window in (200, 640, 5000):
        word.fill_(window)
        for basic in (False, True):
            want, want_lse = c.attn_fwd(q, k, v, min(window, t), d ** -0.5, 0.0, None, False, basic)
            got, got_lse = c.attn_fwd(q, k, v, t, d ** -0.5, 0.0, None, False, basic, word)      # the host value is ignored
            assert torch.equal(got, want) and torch.equal(got_lse, want_lse)
            g = torch.randn_like(want)
            grads = []
            for kwargs in ({}, {"window_tensor": word}):
                dk, dv = torch.empty_like(k), torch.empty_like(v)
                dq = c.attn_bwd(q, k, v, want, g, want_lse, dk, dv, min(window, t) if not kwargs else t, d ** -0.5, 0.0, None, basic, **kwargs)
                grads.append((dq, dk.clone(), dv.clone()))
            for a_, b_ in zip(grads[0], grads[1]):
                assert rel(a_, b_) < 2e-3
    ops.check_status()
