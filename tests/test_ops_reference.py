"""Properties of the plain-PyTorch op definitions that everything else is tested against."""
import torch

from gpt_moe_b200.ops import api
from gpt_moe_b200.ops import reference as ref


def test_counted_routing_is_stable_and_consistent():
    torch.manual_seed(0)
    idx = torch.randint(0, 5, (97, 2))
    experts, order, inverse, offsets = ref.counted_expert_routing(idx, 6)
    flat = idx.reshape(-1)
    assert torch.equal(experts, flat[order]) and torch.equal(order[inverse], torch.arange(flat.numel()))
    assert offsets.dtype == torch.int32 and offsets[-1] == flat.numel() and offsets[4] == offsets[5]      # expert 5 empty
    start = 0
    for e, end in enumerate(offsets.tolist()):
        seg = order[start:end]
        assert torch.all(flat[seg] == e) and torch.all(seg[1:] > seg[:-1])    # original order kept inside a bucket
        start = end


def test_attention_window_is_inclusive_and_padding_rows_are_zero():
    q = k = torch.zeros(1, 6, 1, 4)
    v = torch.arange(6.0).view(1, 6, 1, 1).expand(1, 6, 1, 4).contiguous()
    out = ref.attention(q, k, v, causal=True, window=2)
    # uniform scores: row i averages keys max(0, i-2)..i  (W+1 = 3 keys)
    assert torch.allclose(out[0, :, 0, 0], torch.tensor([0.0, 0.5, 1.0, 2.0, 3.0, 4.0]))
    mask = torch.tensor([[True, True, True, True, False, False]])
    out = ref.attention(q, k, v, causal=True, window=None, attn_mask=mask)
    assert torch.all(out[0, 4:] == 0)
    docs = torch.tensor([[0, 0, 0, 1, 1, 1]])
    out = ref.attention(q, k, v, causal=True, window=None, document_ids=docs)
    assert torch.allclose(out[0, 3:, 0, 0], torch.tensor([3.0, 3.5, 4.0]))


def test_softcap_variants_agree_near_zero_and_saturate():
    s = torch.linspace(-60, 60, 101)
    for backend in ("exact", "ptx", "rational", "clamp"):
        y = ref.softcap(s, 15.0, backend)
        assert y.abs().max() <= 15.0 + 1e-5
        assert abs(y[50].item()) < 1e-4
    small = torch.linspace(-2, 2, 9)
    assert torch.allclose(ref.softcap(small, 15.0, "rational"), ref.softcap(small, 15.0, "exact"), atol=3e-3)


def test_rope_is_a_rotation_of_interleaved_pairs():
    torch.manual_seed(1)
    x = torch.randn(2, 5, 3, 8)
    cos, sin = ref.rope_tables(8, 10000.0, 5)
    y = ref.apply_rope(x, cos, sin)
    assert torch.allclose(y.pow(2).sum(-1), x.pow(2).sum(-1), atol=1e-5)
    assert torch.allclose(y[:, 0], x[:, 0])                       # position 0: identity
    theta = 1.0                                                      # first pair rotates by position * 1
    assert torch.allclose(y[0, 1, 0, 0], x[0, 1, 0, 0] * torch.cos(torch.tensor(theta)) - x[0, 1, 0, 1] * torch.sin(torch.tensor(theta)), atol=1e-6)


def test_qk_norm_clamps_scale_and_blocks_its_gradient():
    x = torch.randn(1, 3, 2, 16)
    scale = torch.tensor([2.0, 7.0]).view(1, 2, 1, 1).requires_grad_()
    y = ref.qk_norm(x, scale, 1e-6, True, float("-inf"), 5.0)
    rms = y.pow(2).mean(-1).sqrt()
    assert torch.allclose(rms[..., 0], torch.full_like(rms[..., 0], 2.0), atol=1e-3)
    assert torch.allclose(rms[..., 1], torch.full_like(rms[..., 1], 5.0), atol=1e-3)
    y.sum().backward()
    assert scale.grad.view(-1)[1] == 0


def test_e8m0_scale_rule_and_mxfp8_roundtrip():
    amax = torch.tensor([0.0, 448.0, 449.0, 1.0, 2 ** -140, float("inf"), float("nan")])
    s = ref.e8m0_scale_from_amax(amax)
    assert s[0] == 1.0 and s[1] == 1.0 and s[2] == 2.0 and s[3] == 2.0 ** -8
    assert s[4] == 2.0 ** -126 and s[5] == 0.0 and s[6] == 0.0
    x = torch.randn(4, 64) * torch.tensor([1e-3, 1.0, 30.0, 1e4]).view(4, 1)
    q, sc = ref.mxfp8_quantize(x)
    assert q.dtype == torch.float8_e4m3fn and sc.shape == (4, 2)
    assert torch.all(torch.log2(sc) == torch.log2(sc).round())     # powers of two
    back = ref.mxfp8_dequantize(q, sc)
    assert ((back - x).abs() / x.abs().clamp(min=1e-9)).median() < 0.05
    tall = torch.randn(64, 8)
    assert torch.equal(ref.mxfp8_roundtrip(tall, 0), ref.mxfp8_roundtrip(tall.t().contiguous(), 1).t())


def test_mxfp8_linear_emulation_gradients_are_close_to_exact():
    torch.manual_seed(2)
    x = torch.randn(40, 96, requires_grad=True)
    w = torch.randn(48, 96, requires_grad=True)
    y = api.linear(x, w, None, "mxfp8")
    y.backward(torch.ones_like(y))
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    y2 = api.linear(x2, w2, None, "default")
    y2.backward(torch.ones_like(y2))
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()
    assert rel(y, y2) < 0.05 and rel(x.grad, x2.grad) < 0.06 and rel(w.grad, w2.grad) < 0.06


def test_polar_express_orthogonalises_and_backends_agree():
    torch.manual_seed(3)
    g = torch.randn(48, 96)
    o = ref.polar_express(g, dtype=torch.float32)
    sv = torch.linalg.svdvals(o)
    assert sv.max() < 1.25 and sv.min() > 0.6
    exact = ref.svd_orthogonalize(g)
    assert ((o - exact).norm() / exact.norm()) < 0.25
    tall = ref.polar_express(g.t().contiguous(), dtype=torch.float32)
    assert torch.allclose(tall, o.t(), atol=1e-4)
    ns = ref.newton_schulz5(g, steps=8, dtype=torch.float32)
    assert torch.linalg.svdvals(ns).max() < 1.3


def test_moe_experts_matches_dense_evaluation():
    torch.manual_seed(4)
    m, d, h, e, k = 50, 16, 24, 4, 2
    hidden = torch.randn(m, d)
    logits = torch.randn(m, e)
    idx, gates, probs = ref.router_gates(logits, k, False)
    assert torch.allclose(gates.sum(-1), torch.ones(m))
    ups = [torch.randn(2 * h, d) for _ in range(e)]
    downs = [torch.randn(d, h) for _ in range(e)]
    out = api.moe_experts(hidden, idx, gates, ups, downs, None, None, "swiglu", "default", "default")
    want = torch.zeros(m, d)
    for t in range(m):
        for s in range(k):
            ex = idx[t, s].item()
            want[t] += gates[t, s] * (ref.activate(hidden[t] @ ups[ex].t(), "swiglu") @ downs[ex].t())
    assert torch.allclose(out, want, atol=1e-4)
    _, g1, p1 = ref.router_gates(logits, 1, False)
    assert torch.allclose(g1[:, 0], p1.max(-1).values)       # top-1 gate = full-softmax probability, not 1.0
    loss = ref.load_balance_loss(torch.full((m, e), 1 / e), torch.arange(m)[:, None] % e, e)
    assert abs(loss.item() - 1.0) < 0.05                     # perfectly balanced routing gives 1


def test_document_starts_reproduce_the_document_mask():
    """The GPU kernels fold document masking into a per-row look-back bound; that bound must describe the same mask as
    comparing document ids pairwise (documents are contiguous runs of tokens)."""
    from gpt_moe_b200.ops.attention_tc import document_starts
    torch.manual_seed(0)
    b, t, window = 3, 97, 20
    ends = (torch.rand(b, t) < 0.08).long()
    docs = ends.cumsum(dim=1) - ends
    starts = document_starts(docs)
    keep = ref.attention_mask(t, "cpu", True, window, None, docs)                  # [B, 1, T, T] or broadcastable
    q = torch.arange(t)[None, :, None]
    k = torch.arange(t)[None, None, :]
    lo = torch.maximum(q - window, starts[:, :, None].long())
    want = (k <= q) & (k >= lo)
    assert torch.equal(keep.reshape(b, t, t) if keep.dim() == 4 else keep.expand(b, t, t), want)
